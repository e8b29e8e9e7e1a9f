"""Configuration: keys, defaults, refusals, registry, model plan."""

import json

import pytest

import tiny
from freetoken_b200.config.minimax_m3 import ConfigError, MiniMaxM3Config, build_plan, rename_checkpoint_tensor
from freetoken_b200.config.model_plan import ModelPlan, RunEntry, schedule_from_lists
from freetoken_b200.registry import architecture_of, get_architecture, known_architectures, read_model_config


def test_reads_every_key_of_the_tiny_configs():
    a = MiniMaxM3Config.from_dict(tiny.TINY_A)
    assert (a.hidden_size, a.num_hidden_layers, a.num_attention_heads, a.num_key_value_heads) == (64, 2, 4, 2)
    assert (a.head_dim, a.rotary_dim, a.rope_theta) == (16, 8, 10000.0)
    assert (a.use_qk_norm, a.qk_norm_type, a.use_gemma_norm) == (True, "per_layer", False)
    assert (a.num_local_experts, a.num_experts_per_tok, a.intermediate_size) == (4, 2, 32)
    assert (a.scoring_func, a.use_routing_bias, a.norm_topk_prob, a.routed_scaling_factor) == ("sigmoid", True, True, 1.0)
    assert (a.vocab_size, a.tie_word_embeddings, a.rms_norm_eps) == (256, False, 1e-6)
    assert (a.q_size, a.kv_size, a.group, a.sm_scale) == (64, 32, 2, 0.25)
    b = MiniMaxM3Config.from_dict(tiny.TINY_B)
    assert (b.head_dim, b.rotary_dim, b.scoring_func, b.norm_topk_prob) == (24, 24, "softmax", False)
    assert b.tie_word_embeddings and not b.use_qk_norm and b.hidden_act == "swigluoai"


def test_defaults_follow_the_reference_readers():
    raw = dict(hidden_size=64, num_hidden_layers=1, num_attention_heads=4, vocab_size=10,
               max_position_embeddings=32, rms_norm_eps=1e-5, num_local_experts=2,
               num_experts_per_tok=1, intermediate_size=8, architectures=["MiniMaxM3ForCausalLM"])
    c = MiniMaxM3Config.from_dict(raw)
    assert c.head_dim == 16 and c.num_key_value_heads == 4          # hidden // heads; kv = q heads
    assert c.rotary_dim == 16 and c.rope_theta == 10000.0           # factor 1.0; default base
    assert c.use_qk_norm and c.qk_norm_type == "per_head" and c.use_gemma_norm
    assert c.scoring_func == "sigmoid" and c.norm_topk_prob and not c.use_routing_bias
    assert c.routed_scaling_factor == 1.0 and c.hidden_act == "swigluoai" and not c.tie_word_embeddings
    half = MiniMaxM3Config.from_dict({**raw, "partial_rotary_factor": 0.5})
    assert half.rotary_dim == 8
    nested = MiniMaxM3Config.from_dict({"architectures": raw["architectures"],
                                        "text_config": {**raw, "rope_parameters": {"rope_theta": 5e6}}})
    assert nested.rope_theta == 5e6


@pytest.mark.parametrize("change,needle", [
    ({"hidden_size": None}, "hidden_size"),
    ({"num_key_value_heads": 3}, "num_key_value_heads"),
    ({"rotary_dim": 7}, "rotary_dim"),
    ({"rotary_dim": 32}, "rotary_dim"),
    ({"num_experts_per_tok": 9}, "num_experts_per_tok"),
    ({"scoring_func": "tanh"}, "scoring_func"),
    ({"qk_norm_type": "per_token"}, "qk_norm_type"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 4}}, "rope_scaling"),
    ({"sparse_attention_config": {"use_sparse_attention": True}}, "sparse_attention"),
    ({"n_shared_experts": 1}, "n_shared_experts"),
    ({"moe_layer_freq": [0, 1]}, "moe_layer_freq"),
    ({"quantization_config": {"quant_method": "fp8"}}, "quantization_config"),
    ({"attention_output_gate": True}, "attention_output_gate"),
])
def test_bad_or_foreign_keys_are_refused_by_name(change, needle):
    with pytest.raises(ConfigError) as err:
        MiniMaxM3Config.from_dict({**tiny.TINY_A, **change})
    assert needle in str(err.value)


def test_registry_maps_names_to_the_architecture(tmp_path):
    for name in ("MiniMaxM3ForCausalLM", "MiniMaxM3SparseForCausalLM", "MiniMaxM3SparseForConditionalGeneration"):
        assert name in known_architectures()
        assert get_architecture(name).build_plan is build_plan
    with pytest.raises(ValueError, match="not supported"):
        get_architecture("LlamaForCausalLM")
    with pytest.raises(ValueError, match="architectures"):
        architecture_of({"hidden_size": 1})
    (tmp_path / "config.json").write_text(json.dumps(tiny.TINY_B))
    arch, cfg = read_model_config(str(tmp_path))
    assert arch.name == "MiniMaxM3ForCausalLM" and cfg.num_hidden_layers == 3


def test_plan_carries_every_size_as_a_parameter():
    cfg = MiniMaxM3Config.from_dict(tiny.TINY_C)
    plan = build_plan(cfg)
    assert len(plan.layers) == 2 and [s.layer for s in plan.schedule] == [0, 1]
    mixer = plan.layers[0].mixer
    assert mixer.kind == "paged_attention" and mixer.params["num_heads"] == 12
    assert mixer.params["qk_norm"] == "per_head" and mixer.params["position"].params["rotary_dim"] == 16
    ffn = plan.layers[1].feed_forward
    assert ffn.params["num_experts"] == 16 and ffn.params["scale"] == 2.0 and ffn.params["use_bias"]
    assert plan.head.params["tied_to"] is None
    tied = build_plan(MiniMaxM3Config.from_dict(tiny.TINY_B))
    assert tied.head.params["tied_to"] == "model.embed_tokens.weight"
    assert tied.layers[0].mixer.params["qk_norm"] == "none"


def test_schedule_rules():
    cfg = MiniMaxM3Config.from_dict(tiny.TINY_A)
    plan = build_plan(cfg)

    def with_schedule(s):
        return ModelPlan(**{**plan.__dict__, "schedule": s})

    with_schedule(schedule_from_lists([0, 1, 0])).validate()                 # a layer twice
    with_schedule(schedule_from_lists([0, 1], {1: 0})).validate()            # stop 1 reads stop 0's cache
    with pytest.raises(ValueError, match="outside"):
        with_schedule((RunEntry(5),)).validate()
    with pytest.raises(ValueError, match="does not run before"):
        with_schedule(schedule_from_lists([0, 1], {0: 1})).validate()
    with pytest.raises(ValueError, match="no cache of its own"):
        with_schedule(schedule_from_lists([0, 1, 0], {1: 0, 2: 1})).validate()


def test_checkpoint_names():
    assert rename_checkpoint_tensor("language_model.model.layers.0.self_attn.q_proj.weight") == \
        "model.layers.0.self_attn.q_proj.weight"
    assert rename_checkpoint_tensor("model.norm.weight") == "model.norm.weight"
    assert rename_checkpoint_tensor("vision_tower.blocks.0.attn.qkv.weight") is None
    assert rename_checkpoint_tensor("model.layers.1.self_attn.k_proj.k_scale") is None
