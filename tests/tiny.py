"""Tiny configurations of the architecture and helpers that tests share.

tiny-A and tiny-B differ in every size and option: head counts and group size,
head size (16 vs 24, the latter no power of two), rotary span (partial vs
full), theta, QK norm (per layer vs none), norm form (plain vs 1+w) and eps,
experts / top-k / expert width, scoring (sigmoid+bias+renormalised vs softmax
without either), routed scaling factor, activation, vocabulary and tied head,
number of layers.  tiny-C adds the per-head QK norm and a head size the
tensor-core kernels take.
"""

from __future__ import annotations

from typing import Dict, List

import torch

TINY_A: Dict = dict(
    architectures=["MiniMaxM3ForCausalLM"], model_type="minimax_m3",
    hidden_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
    head_dim=16, rotary_dim=8, rope_theta=10000.0, max_position_embeddings=512,
    rms_norm_eps=1e-6, use_gemma_norm=False, use_qk_norm=True, qk_norm_type="per_layer",
    num_local_experts=4, num_experts_per_tok=2, intermediate_size=32,
    scoring_func="sigmoid", use_routing_bias=True, norm_topk_prob=True,
    routed_scaling_factor=1.0, hidden_act="silu", vocab_size=256, tie_word_embeddings=False,
)

TINY_B: Dict = dict(
    architectures=["MiniMaxM3ForCausalLM"], model_type="minimax_m3",
    hidden_size=96, num_hidden_layers=3, num_attention_heads=6, num_key_value_heads=3,
    head_dim=24, rotary_dim=24, rope_theta=1e6, max_position_embeddings=512,
    rms_norm_eps=1e-5, use_gemma_norm=True, use_qk_norm=False,
    num_local_experts=8, num_experts_per_tok=3, intermediate_size=48,
    scoring_func="softmax", use_routing_bias=False, norm_topk_prob=False,
    routed_scaling_factor=1.5, hidden_act="swigluoai", swiglu_alpha=1.702, swiglu_limit=7.0,
    vocab_size=384, tie_word_embeddings=True,
)

TINY_C: Dict = dict(
    architectures=["MiniMaxM3SparseForCausalLM"], model_type="minimax_m3",
    hidden_size=128, num_hidden_layers=2, num_attention_heads=12, num_key_value_heads=2,
    head_dim=32, rotary_dim=16, rope_theta=5e6, max_position_embeddings=1024,
    rms_norm_eps=1e-6, use_gemma_norm=True, use_qk_norm=True, qk_norm_type="per_head",
    num_local_experts=16, num_experts_per_tok=4, intermediate_size=64,
    scoring_func="sigmoid", use_routing_bias=True, norm_topk_prob=True,
    routed_scaling_factor=2.0, hidden_act="silu", vocab_size=500, tie_word_embeddings=False,
)

# Awkward sizes on purpose: a width and a vocabulary that are no power of two,
# one query head per KV head, a head size of 48 with 20 rotary dims, every
# expert chosen for every token, an expert width that is no multiple of 16.
TINY_D: Dict = dict(
    architectures=["MiniMaxM3ForCausalLM"], model_type="minimax_m3",
    hidden_size=200, num_hidden_layers=2, num_attention_heads=5, num_key_value_heads=5,
    head_dim=48, rotary_dim=20, rope_theta=123456.0, max_position_embeddings=300,
    rms_norm_eps=3e-6, use_gemma_norm=False, use_qk_norm=True, qk_norm_type="per_head",
    num_local_experts=5, num_experts_per_tok=5, intermediate_size=40,
    scoring_func="sigmoid", use_routing_bias=False, norm_topk_prob=False,
    routed_scaling_factor=0.5, hidden_act="silu", vocab_size=333, tie_word_embeddings=True,
)

# Head size 64 and pages of 64 tokens: what the tcgen05 prefill attention takes.
TINY_E: Dict = dict(
    architectures=["MiniMaxM3ForCausalLM"], model_type="minimax_m3",
    hidden_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
    head_dim=64, rotary_dim=32, rope_theta=10000.0, max_position_embeddings=1024,
    rms_norm_eps=1e-5, use_gemma_norm=False, use_qk_norm=True, qk_norm_type="per_layer",
    num_local_experts=6, num_experts_per_tok=2, intermediate_size=48,
    scoring_func="softmax", use_routing_bias=False, norm_topk_prob=True,
    routed_scaling_factor=1.0, hidden_act="silu", vocab_size=320, tie_word_embeddings=False,
)

# Sizes between the kernels' fast shapes: a head size of 80 (a step of 16 that no
# tensor-core kernel takes), seven query heads per KV head, 40 of 48 experts per token
# (more choices than a warp has lanes), a page of 12 tokens.
TINY_F: Dict = dict(
    architectures=["MiniMaxM3ForCausalLM"], model_type="minimax_m3",
    hidden_size=112, num_hidden_layers=2, num_attention_heads=7, num_key_value_heads=1,
    head_dim=80, rotary_dim=48, rope_theta=25000.0, max_position_embeddings=256,
    rms_norm_eps=2e-6, use_gemma_norm=True, use_qk_norm=True, qk_norm_type="per_layer",
    num_local_experts=48, num_experts_per_tok=40, intermediate_size=24,
    scoring_func="sigmoid", use_routing_bias=True, norm_topk_prob=True,
    routed_scaling_factor=1.25, hidden_act="swigluoai", vocab_size=211, tie_word_embeddings=False,
)

TINY = {"A": TINY_A, "B": TINY_B, "C": TINY_C, "D": TINY_D, "E": TINY_E, "F": TINY_F}
SEEDS = {"A": 0, "B": 1, "C": 2, "D": 3, "E": 4, "F": 5}
PAGE = {"A": 4, "B": 8, "C": 16, "D": 32, "E": 64, "F": 12}


def random_options(which: str):
    from freetoken_b200.weights import RandomOptions
    if which == "A":
        return RandomOptions(norm_std=0.0, router_bias_std=0.01)
    if which == "B":
        return RandomOptions(norm_std=0.1)
    if which in ("D", "E"):
        return RandomOptions(norm_std=0.1)
    if which == "F":
        return RandomOptions(norm_std=0.05, router_bias_std=0.2)
    return RandomOptions(norm_std=0.05, router_bias_std=0.05)


def write_tiny(folder: str, which: str, file_dtype=torch.bfloat16, config: Dict = None) -> str:
    """Write the tiny model ``which`` into ``folder`` with the framework's
    random-weights mode; returns the folder."""
    from freetoken_b200.models import Model
    from freetoken_b200.registry import architecture_of
    from freetoken_b200.weights import write_model_folder

    config = dict(config or TINY[which])
    arch = architecture_of(config)
    model = Model(arch.build_plan(arch.read_config(config)))
    write_model_folder(folder, config, model.tensor_specs(), SEEDS[which], file_dtype,
                       random_options(which))
    return folder


def tokens(seed: int, n: int, vocab: int) -> List[int]:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


# Tolerances, fixed up front.  float32: the engine and the plain implementation
# sum in different orders; logits of these models are O(0.1..1).  bfloat16:
# every stored activation carries a relative rounding error of 2^-9.
TOL = {"float32": dict(atol=2e-5, rtol=1e-4), "bfloat16": dict(atol=2e-2, rtol=2e-2)}
