"""More generality of the parts, again with parts defined HERE in the test and
no change to the framework's files: another position encoding (a rotary whose
angle grows with the square root of the position, used by the framework's own
attention mixer and kernels), a feed-forward with a routing of its own (the
token id's parity of the strongest input feature picks one of three plain MLPs)
and a norm of its own (LayerNorm without bias) - registered, built from a model
folder, stepped whole, in portions and in mixed batches, and compared with a
plain implementation written beside it.  None of this is a model of anyone's."""

import os
from dataclasses import dataclass
from typing import List

import pytest
import torch

import plain_model as pm
import replay_driver as rd
import tiny

pytestmark = pytest.mark.gpu

H, V, NQ, NKV, D, R, E, I = 40, 90, 6, 3, 16, 16, 3, 56
EPS = 1e-5
TOY = dict(architectures=["ToyPartsForCausalLM"], hidden=H, vocab=V)


def sqrt_rotary_table(positions: int) -> torch.Tensor:
    """[positions, R]: cos | sin of sqrt(p) * 3^(-2i/R)."""
    inv = 1.0 / (3.0 ** (torch.arange(0, R, 2, dtype=torch.float) / R))
    ang = torch.arange(positions, dtype=torch.float).sqrt()[:, None] * inv[None, :]
    return torch.cat((ang.cos(), ang.sin()), -1).contiguous()


def register_toy_parts():
    from freetoken_b200.config.model_plan import LayerSpec, ModelPlan, PartSpec, sequential_schedule
    from freetoken_b200.parts import (FeedForward, Norm, Position, register_feed_forward, register_norm,
                                      register_position)
    from freetoken_b200.registry import Architecture, register_architecture
    from freetoken_b200.weights import Init, TensorSpec

    @register_position("toy_sqrt_rotary")
    class SqrtRotary(Position):
        """What the attention mixer reads from a position encoding: a table of
        cos | sin per position, how many dims rotate, and the pairing."""
        interleaved = False
        rotary_dim = R

        def table(self, device, positions: int):
            return sqrt_rotary_table(min(positions, 512)).to(device)

    @register_norm("toy_layernorm")
    class LayerNormNoBias(Norm):
        def __init__(self, spec, prefix):
            super().__init__(spec, prefix)
            self.n_w = self.name(spec.params["scope"] + ".weight")
            self.w = None

        def tensor_specs(self):
            return [TensorSpec(self.n_w, (H,), role="small32", init=Init(mean=1.0, std=0.1))]

        def bind(self, tensors, dtype):
            self.w = tensors[self.n_w]

        def forward(self, ctx, delta, residual):
            if delta is not None:
                residual.add_(delta.float() if delta.dim() == 2 else delta.float().sum(1))
            mu = residual.mean(-1, keepdim=True)
            var = ((residual - mu) ** 2).mean(-1, keepdim=True)
            return ((residual - mu) * torch.rsqrt(var + EPS) * self.w).to(ctx.dtype)

    @register_feed_forward("toy_argmax_mlps")
    class ArgmaxMlps(FeedForward):
        """expert = argmax(|x|) mod E; y = W2[e] tanh(W1[e] x).  Routing by the
        input alone: no router weights, one expert per token."""

        def __init__(self, spec, prefix):
            super().__init__(spec, prefix)
            self.n1, self.n2 = self.name("ff.w1"), self.name("ff.w2")
            self.w1 = self.w2 = None

        def tensor_specs(self):
            return [TensorSpec(self.n1, (E, I, H)), TensorSpec(self.n2, (E, H, I))]

        def bind(self, tensors, dtype):
            self.w1, self.w2 = tensors[self.n1], tensors[self.n2]

        def forward(self, ctx, x):
            e = x.float().abs().argmax(-1) % E
            mid = torch.tanh(torch.einsum("tih,th->ti", self.w1[e].float(), x.float()))
            return torch.einsum("thi,ti->th", self.w2[e].float(), mid).to(x.dtype)

    @dataclass(frozen=True)
    class Cfg:
        hidden: int
        vocab: int

    def build_plan(cfg: Cfg) -> ModelPlan:
        def norm(scope):
            return PartSpec("toy_layernorm", {"scope": scope})

        attention = PartSpec("paged_attention", {
            "hidden_size": H, "num_heads": NQ, "num_kv_heads": NKV, "head_dim": D, "sm_scale": 0.3,
            "qk_norm": "none", "sliding_window": None, "position": PartSpec("toy_sqrt_rotary", {}),
            "scope": "attn",
            "checkpoint_names": {"qkv": "qkv.weight", "o": "o.weight", "q": "q.weight", "k": "k.weight",
                                 "v": "v.weight", "q_norm": "qn.weight", "k_norm": "kn.weight"}})
        layers = tuple(LayerSpec(f"blocks.{i}", PartSpec("prenorm", {}), attention,
                                 PartSpec("toy_argmax_mlps", {}), norm("n1"), norm("n2")) for i in range(2))
        return ModelPlan("ToyPartsForCausalLM", H, V,
                         PartSpec("token_embedding", {"vocab_size": V, "hidden_size": H, "prefix": "",
                                                      "scope": "embed"}),
                         layers, sequential_schedule(2),
                         PartSpec("toy_layernorm", {"scope": "final_norm", "prefix": ""}),
                         PartSpec("lm_head", {"vocab_size": V, "hidden_size": H, "prefix": "", "scope": "head",
                                              "tied_to": None}),
                         512)

    return register_architecture(Architecture(
        name="ToyPartsForCausalLM", read_config=lambda raw: Cfg(raw["hidden"], raw["vocab"]),
        build_plan=build_plan, config_to_dict=lambda cfg: dict(TOY)))


# ------------------------------------------------- the plain implementation of it
def layernorm(x, w):
    mu = x.mean(-1, keepdim=True)
    return (x - mu) * torch.rsqrt(((x - mu) ** 2).mean(-1, keepdim=True) + EPS) * w


def neox(x, cos, sin):
    half = R // 2
    x1, x2 = x[..., :half], x[..., half:R]
    c, s = cos[:, None, :], sin[:, None, :]
    return torch.cat((x1 * c - x2 * s, x2 * c + x1 * s, x[..., R:]), -1)


def plain_forward(folder: str, tokens: List[int]) -> torch.Tensor:
    t = {k: v.float() for k, v in pm.read_safetensors(os.path.join(folder, "model.safetensors")).items()}
    T = len(tokens)
    table = sqrt_rotary_table(T)
    cos, sin = table[:, :R // 2], table[:, R // 2:]
    residual = t["embed.weight"][torch.tensor(tokens)]
    x = torch.zeros_like(residual)
    for i in range(2):
        p = f"blocks.{i}"
        residual = residual + x
        h = layernorm(residual, t[f"{p}.n1.weight"])
        q = neox((h @ t[f"{p}.attn.q.weight"].t()).view(T, NQ, D), cos, sin)
        k = neox((h @ t[f"{p}.attn.k.weight"].t()).view(T, NKV, D), cos, sin)
        v = (h @ t[f"{p}.attn.v.weight"].t()).view(T, NKV, D)
        o = pm.causal_attention(q, k, v, 0.3, None)
        residual = residual + o.reshape(T, NQ * D) @ t[f"{p}.attn.o.weight"].t()
        h = layernorm(residual, t[f"{p}.n2.weight"])
        e = h.abs().argmax(-1) % E
        mid = torch.tanh(torch.einsum("tih,th->ti", t[f"{p}.ff.w1"][e], h))
        x = torch.einsum("thi,ti->th", t[f"{p}.ff.w2"][e], mid)
    return layernorm(residual + x, t["final_norm.weight"]) @ t["head.weight"].t()


# ------------------------------------------------------------------------- tests
@pytest.fixture(scope="module")
def toy_folder(tmp_path_factory):
    from freetoken_b200.models import Model
    from freetoken_b200.weights import RandomOptions, write_model_folder
    arch = register_toy_parts()
    folder = str(tmp_path_factory.mktemp("toyparts"))
    model = Model(arch.build_plan(arch.read_config(TOY)))
    write_model_folder(folder, TOY, model.tensor_specs(), 11, torch.float32,
                       RandomOptions(matrix_std=0.1, norm_std=0.1))
    return folder


@pytest.mark.parametrize("cut", ["whole", "decode_tail", "portions", "mixed"])
def test_toy_parts_step_like_their_plain_implementation(toy_folder, cut):
    from freetoken_b200.engine import Engine, EngineArgs
    reqs = {f"r{i}": tiny.tokens(70 + i, n, V) for i, n in enumerate([2, 33, 19, 48])}
    fn = {"whole": rd.whole, "decode_tail": lambda r: rd.decode_tail(r, 7), "portions": rd.portions,
          "mixed": rd.mixed}[cut]
    schedule = fn(reqs)
    engine = Engine.from_folder(toy_folder, EngineArgs(dtype="float32", page_size=8,
                                                       num_pages=-(-rd.peak_tokens(schedule, 8) // 8),
                                                       max_running_requests=4))
    got = rd.run_engine(engine, reqs, schedule)
    for rid, toks in reqs.items():
        want = plain_forward(toy_folder, toks)
        assert torch.allclose(got[rid], want, atol=5e-5, rtol=1e-4), (cut, rid, (got[rid] - want).abs().max())
    assert engine.cache.free_pages() == engine.cache.total_pages()
