"""Generality of the parts: an architecture defined HERE, in the test, with a
mixer that keeps a state of its own, a layer that runs twice, a stop that reads
another stop's cache and a windowed attention layer, is registered, built from a
model folder and stepped - whole, in portions and in mixed batches - without a
change to any file of the framework, and agrees with a plain implementation
written beside it."""

import os
from dataclasses import dataclass
from typing import List

import pytest
import torch

import plain_model as pm
import replay_driver as rd
import tiny

pytestmark = pytest.mark.gpu

H, V, NQ, NKV, D, E, K, I = 48, 120, 4, 2, 16, 4, 2, 24
WINDOW = 6
TOY = dict(architectures=["ToyStateForCausalLM"], hidden=H, vocab=V, decay=0.75)


# ---------------------------------------------------------------- the toy parts
def register_toy():
    from freetoken_b200.cache import StateNeed
    from freetoken_b200.config.model_plan import (LayerSpec, ModelPlan, PartSpec, RunEntry)
    from freetoken_b200.parts import Mixer, register_mixer
    from freetoken_b200.registry import Architecture, register_architecture
    from freetoken_b200.weights import TensorSpec

    @register_mixer("toy_decaying_sum")
    class DecayingSum(Mixer):
        """y_t = (s_t) W with s_t = decay * s_{t-1} + x_t: a state of fixed size
        per request, carried from step to step in a state slot."""

        def __init__(self, spec, prefix):
            super().__init__(spec, prefix)
            self.hidden = spec.params["hidden"]
            self.decay = spec.params["decay"]
            self.n_w = self.name("mix.weight")
            self.w = None

        def cache_need(self):
            return StateNeed((self.hidden,), "float32")

        def tensor_specs(self):
            return [TensorSpec(self.n_w, (self.hidden, self.hidden))]

        def bind(self, tensors, dtype):
            self.w = tensors[self.n_w]

        def forward(self, ctx, x, cache):
            out = torch.empty_like(x)
            for seg in ctx.segments:                     # tokens of a request in order, exactly once
                s = cache.state[seg.slot]
                for r in range(seg.q_start, seg.q_start + seg.n):
                    s.mul_(self.decay).add_(x[r].float())
                    out[r] = (s @ self.w.float().t()).to(x.dtype)
            return out

    @dataclass(frozen=True)
    class ToyConfig:
        hidden: int
        vocab: int
        decay: float

    def build_plan(cfg: ToyConfig) -> ModelPlan:
        def norm(scope):
            return PartSpec("rmsnorm", {"size": cfg.hidden, "eps": 1e-5, "plus_one": False, "scope": scope})

        def attention(window):
            return PartSpec("paged_attention", {
                "hidden_size": cfg.hidden, "num_heads": NQ, "num_kv_heads": NKV, "head_dim": D,
                "sm_scale": D ** -0.5, "qk_norm": "per_head", "qk_norm_eps": 1e-5,
                "qk_norm_plus_one": False, "sliding_window": window,
                "position": PartSpec("rotary_interleaved", {"head_dim": D, "rotary_dim": 8, "theta": 1e4,
                                                            "max_position": 256}),
                "scope": "attn",
                "checkpoint_names": {"qkv": "qkv.weight", "o": "o.weight", "q": "q.weight", "k": "k.weight",
                                     "v": "v.weight", "q_norm": "qn.weight", "k_norm": "kn.weight"}})

        ffn = PartSpec("routed_experts", {
            "hidden_size": cfg.hidden, "intermediate_size": I, "num_experts": E, "top_k": K,
            "scoring": "softmax", "use_bias": False, "renormalize": True, "scale": 1.0,
            "activation": "silu", "scope": "moe",
            "checkpoint_names": {"router": "router.weight", "bias": "router.bias", "gate_up": "gate_up",
                                 "down": "down", "gate": "e{e}.gate.weight", "up": "e{e}.up.weight",
                                 "down_each": "e{e}.down.weight"}})
        toy = PartSpec("toy_decaying_sum", {"hidden": cfg.hidden, "decay": cfg.decay})

        def layer(i, mixer):
            return LayerSpec(f"blocks.{i}", PartSpec("prenorm", {}), mixer, ffn, norm("n1"), norm("n2"))

        layers = (layer(0, toy), layer(1, attention(None)), layer(2, attention(WINDOW)))
        # layer 0 runs twice (a state per stop); the last stop runs layer 1
        # again on the cache that stop 1 wrote
        schedule = (RunEntry(0), RunEntry(1), RunEntry(0), RunEntry(2), RunEntry(1, reads_cache_of=1))
        return ModelPlan("ToyStateForCausalLM", cfg.hidden, cfg.vocab,
                         PartSpec("token_embedding", {"vocab_size": cfg.vocab, "hidden_size": cfg.hidden,
                                                      "prefix": "", "scope": "embed"}),
                         layers, schedule,
                         PartSpec("rmsnorm", {**norm("final_norm").params, "prefix": ""}),
                         PartSpec("lm_head", {"vocab_size": cfg.vocab, "hidden_size": cfg.hidden,
                                              "prefix": "", "scope": "head", "tied_to": None}),
                         256)

    return register_architecture(Architecture(
        name="ToyStateForCausalLM",
        read_config=lambda raw: ToyConfig(raw["hidden"], raw["vocab"], raw["decay"]),
        build_plan=build_plan,
        config_to_dict=lambda cfg: dict(TOY)))


# ------------------------------------------------- the plain implementation of it
def interleaved_rope(x, cos, sin, R):
    """(2i, 2i+1) pairing, python/freetoken/kernel/triton/rope.py:59-61,73-78."""
    y = x.float().clone()
    x0, x1 = x[..., 0:R:2].float(), x[..., 1:R:2].float()
    c, s = cos[:, None, :], sin[:, None, :]
    y[..., 0:R:2] = x0 * c - x1 * s
    y[..., 1:R:2] = x1 * c + x0 * s
    return y


def plain_forward(folder: str, tokens: List[int]) -> torch.Tensor:
    t = {k: v.float() for k, v in pm.read_safetensors(os.path.join(folder, "model.safetensors")).items()}
    T = len(tokens)
    residual = t["embed.weight"][torch.tensor(tokens)]
    x = torch.zeros_like(residual)
    cos, sin = pm.rope_table(T, 8, 1e4)
    kv_of_stop = {}

    def moe(p, h):
        w, ids = pm.route(h, t[f"{p}.moe.router.weight"], None, K, "softmax", True, 1.0)
        gate_up = [torch.cat([t[f"{p}.moe.e{e}.gate.weight"], t[f"{p}.moe.e{e}.up.weight"]]) for e in range(E)]
        down = [t[f"{p}.moe.e{e}.down.weight"] for e in range(E)]
        return pm.experts(h, w, ids, gate_up, down, "silu", 0, 0, lambda z: z)

    def attention(p, h, window, stop, reads):
        q = h @ t[f"{p}.attn.q.weight"].t()
        k = h @ t[f"{p}.attn.k.weight"].t()
        v = h @ t[f"{p}.attn.v.weight"].t()
        q, k = pm.qk_norm(q, k, t[f"{p}.attn.qn.weight"], t[f"{p}.attn.kn.weight"], "per_head", 1e-5,
                          False, NQ, NKV, D)
        q = interleaved_rope(q.view(T, NQ, D), cos, sin, 8)
        k = interleaved_rope(k.view(T, NKV, D), cos, sin, 8)
        if reads is None:
            kv_of_stop[stop] = (k, v.view(T, NKV, D))
        k, v = kv_of_stop[stop if reads is None else reads]
        o = pm.causal_attention(q, k, v, D ** -0.5, window)
        return o.reshape(T, NQ * D) @ t[f"{p}.attn.o.weight"].t()

    def decaying_sum(p, h):
        s = torch.zeros(H)
        out = torch.empty_like(h)
        for i in range(T):
            s = TOY["decay"] * s + h[i]
            out[i] = s @ t[f"{p}.mix.weight"].t()
        return out

    stops = [(0, "toy", None), (1, "attn", None), (0, "toy", None), (2, "window", None), (1, "attn", 1)]
    for stop, (layer, kind, reads) in enumerate(stops):
        p = f"blocks.{layer}"
        residual = residual + x
        h = pm.rms_norm(residual, t[f"{p}.n1.weight"], 1e-5, False)
        if kind == "toy":
            a = decaying_sum(p, h)
        else:
            a = attention(p, h, WINDOW if kind == "window" else None, stop, reads)
        residual = residual + a
        x = moe(p, pm.rms_norm(residual, t[f"{p}.n2.weight"], 1e-5, False))
    return pm.rms_norm(residual + x, t["final_norm.weight"], 1e-5, False) @ t["head.weight"].t()


# ------------------------------------------------------------------------- tests
@pytest.fixture(scope="module")
def toy_folder(tmp_path_factory):
    from freetoken_b200.models import Model
    from freetoken_b200.weights import RandomOptions, write_model_folder
    arch = register_toy()
    folder = str(tmp_path_factory.mktemp("toy"))
    model = Model(arch.build_plan(arch.read_config(TOY)))
    write_model_folder(folder, TOY, model.tensor_specs(), 5, torch.float32, RandomOptions(matrix_std=0.08, norm_std=0.1))
    return folder


def test_toy_model_is_built_from_its_folder(toy_folder):
    from freetoken_b200.engine import Engine, EngineArgs
    engine = Engine.from_folder(toy_folder, EngineArgs(dtype="float32", page_size=4, max_tokens=64,
                                                       max_running_requests=2))
    cache = engine.cache
    assert [g.stops for g in cache.state_groups] == [[0, 2]]            # a state per stop of the twice-run layer
    assert sorted(g.need.window or 0 for g in cache.paged_groups) == [0, WINDOW]
    assert 4 not in cache.paged_index                                    # the last stop owns no cache
    assert engine.cache_views[4].kv_pages.data_ptr() == engine.cache_views[1].kv_pages.data_ptr()
    assert not engine.cache_views[4].writes


@pytest.mark.parametrize("cut", ["whole", "decode_tail", "portions", "mixed"])
def test_toy_model_steps_like_its_plain_implementation(toy_folder, cut):
    from freetoken_b200.engine import Engine, EngineArgs
    reqs = {f"r{i}": tiny.tokens(40 + i, n, V) for i, n in enumerate([3, 26, 41, 17, 30])}
    fn = {"whole": rd.whole, "decode_tail": lambda r: rd.decode_tail(r, 9), "portions": rd.portions,
          "mixed": rd.mixed}[cut]
    schedule = fn(reqs)
    engine = Engine.from_folder(toy_folder, EngineArgs(dtype="float32", page_size=4,
                                                       num_pages=-(-rd.peak_tokens(schedule, 4) // 4),
                                                       max_running_requests=4))
    got = rd.run_engine(engine, reqs, schedule)
    for rid, toks in reqs.items():
        want = plain_forward(toy_folder, toks)
        assert torch.allclose(got[rid], want, atol=5e-5, rtol=1e-4), (cut, rid, (got[rid] - want).abs().max())
    assert engine.cache.free_pages() == engine.cache.total_pages()


def test_toy_model_runs_in_bfloat16_too(toy_folder):
    """The toy mixer's torch code and the framework's bfloat16 kernels side by side."""
    from freetoken_b200.engine import Engine, EngineArgs
    reqs = {"a": tiny.tokens(1, 20, V), "b": tiny.tokens(2, 9, V)}
    schedule = rd.mixed(reqs)
    engine = Engine.from_folder(toy_folder, EngineArgs(dtype="bfloat16", page_size=8, max_tokens=64,
                                                       max_running_requests=2))
    got = rd.run_engine(engine, reqs, schedule)
    for rid, toks in reqs.items():
        want = plain_forward(toy_folder, toks)
        # loose sanity band: bfloat16 weights and activations against the float32 plain model
        assert (got[rid] - want).abs().max() < 0.15 * want.abs().max()
