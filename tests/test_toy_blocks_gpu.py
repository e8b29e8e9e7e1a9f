"""Three more seams, again with parts defined HERE and no change to the
framework's files: a block with three norms (the mixer's output is normed once
more before it joins the residual), a block without a feed-forward, and a mixer
whose cache is not keys and values but one latent vector per token - a cache
need of its own shape, pooled, paged, freed and reused by the manager like any
other.  Registered, built from a model folder, stepped whole, in portions and in
mixed batches with scarce pages, compared with a plain implementation written
beside it.  None of this is a model of anyone's."""

import os
from dataclasses import dataclass
from typing import List, Optional, Tuple

import pytest
import torch

import plain_model as pm
import replay_driver as rd
import tiny

H, V, NQ, NKV, D, E, K, I, W = 40, 100, 4, 2, 16, 4, 2, 24, 12
EPS = 1e-5
TOY = dict(architectures=["ToyBlocksForCausalLM"], hidden=H, vocab=V)


def register_toy_blocks():
    from freetoken_b200.cache import PerTokenNeed
    from freetoken_b200.config.model_plan import LayerSpec, ModelPlan, PartSpec, sequential_schedule
    from freetoken_b200.parts import Block, Mixer, register_block, register_mixer
    from freetoken_b200.registry import Architecture, register_architecture
    from freetoken_b200.weights import TensorSpec

    @dataclass(frozen=True)
    class LatentNeed(PerTokenNeed):
        """One float32 vector of ``width`` per token: pages are [pages, page_size, width]."""
        width: int
        window: Optional[int] = None
        storage_dtype: Optional[str] = "float32"
        kind: str = "toy_latent"
        page_axis = 0

        def layout(self, pages: int, page_size: int) -> Tuple[int, ...]:
            return (pages, page_size, self.width)

        def elements_per_token(self) -> int:
            return self.width

    @register_mixer("toy_latent_mean")
    class LatentMean(Mixer):
        """c_t = Wc x_t is kept per token; y_t = Wo mean(c_0 .. c_t)."""

        def __init__(self, spec, prefix):
            super().__init__(spec, prefix)
            self.n_c, self.n_o = self.name("lat.c.weight"), self.name("lat.o.weight")
            self.wc = self.wo = None

        def cache_need(self):
            return LatentNeed(W)

        def tensor_specs(self):
            return [TensorSpec(self.n_c, (W, H)), TensorSpec(self.n_o, (H, W))]

        def bind(self, tensors, dtype):
            self.wc, self.wo = tensors[self.n_c].float(), tensors[self.n_o].float()

        def forward(self, ctx, x, cache):
            pages = cache.pages                               # [pages, page_size, W]
            table = ctx.block_tables[cache.block_table_index].cpu()
            P = ctx.page_size
            out = torch.empty_like(x)
            for i, seg in enumerate(ctx.segments):
                c = x[seg.q_start: seg.q_start + seg.n].float() @ self.wc.t()
                for j in range(seg.n):
                    pos = seg.pos0 + j
                    pages[int(table[i, pos // P]), pos % P] = c[j]
                total = seg.pos0 + seg.n
                rows = torch.cat([pages[int(table[i, p])] for p in range(-(-total // P))])[:total]
                means = rows.cumsum(0)[seg.pos0:] / torch.arange(seg.pos0 + 1, total + 1, device=x.device)[:, None]
                out[seg.q_start: seg.q_start + seg.n] = (means @ self.wo.t()).to(x.dtype)
            return out

    @register_block("toy_sandwich")
    class Sandwich(Block):
        """h = n1(residual += delta); a = post(mixer(h)); h = n2(residual += a); ffn(h)."""
        NORM_NAMES = ("mixer", "post_mixer", "feed_forward")

        def forward(self, ctx, delta, residual, cache):
            h = self.norms["mixer"].forward(ctx, delta, residual)
            a = self.mixer.forward(ctx, h, cache)
            scratch = torch.zeros_like(residual)
            a = self.norms["post_mixer"].forward(ctx, a, scratch).clone()     # a norm of the branch alone
            h = self.norms["feed_forward"].forward(ctx, a, residual)
            return self.feed_forward.forward(ctx, h)

    @register_block("toy_mixer_only")
    class MixerOnly(Block):
        """h = n(residual += delta); mixer(h): one norm, no feed-forward."""
        NORM_NAMES = ("mixer",)
        HAS_FEED_FORWARD = False

        def forward(self, ctx, delta, residual, cache):
            return self.mixer.forward(ctx, self.norms["mixer"].forward(ctx, delta, residual), cache)

    @dataclass(frozen=True)
    class ToyConfig:
        hidden: int
        vocab: int

    def build_plan(cfg: ToyConfig) -> ModelPlan:
        def norm(scope):
            return PartSpec("rmsnorm", {"size": cfg.hidden, "eps": EPS, "plus_one": False, "scope": scope})

        attention = PartSpec("paged_attention", {
            "hidden_size": cfg.hidden, "num_heads": NQ, "num_kv_heads": NKV, "head_dim": D,
            "sm_scale": D ** -0.5, "qk_norm": "none", "sliding_window": None,
            "position": PartSpec("rotary_neox", {"head_dim": D, "rotary_dim": 8, "theta": 1e4, "max_position": 256}),
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
        latent = PartSpec("toy_latent_mean", {})
        layers = (
            LayerSpec("blocks.0", PartSpec("toy_sandwich", {}), attention, ffn, norm("n1"), norm("n2"),
                      norms={"post_mixer": norm("n_post")}),
            LayerSpec("blocks.1", PartSpec("toy_mixer_only", {}), latent, mixer_norm=norm("n1")),
            LayerSpec("blocks.2", PartSpec("prenorm", {}), latent, ffn, norm("n1"), norm("n2")),
        )
        return ModelPlan("ToyBlocksForCausalLM", cfg.hidden, cfg.vocab,
                         PartSpec("token_embedding", {"vocab_size": cfg.vocab, "hidden_size": cfg.hidden,
                                                      "prefix": "", "scope": "embed"}),
                         layers, sequential_schedule(3),
                         PartSpec("rmsnorm", {**norm("final_norm").params, "prefix": ""}),
                         PartSpec("lm_head", {"vocab_size": cfg.vocab, "hidden_size": cfg.hidden,
                                              "prefix": "", "scope": "head", "tied_to": None}),
                         256)

    return register_architecture(Architecture(
        name="ToyBlocksForCausalLM",
        read_config=lambda raw: ToyConfig(raw["hidden"], raw["vocab"]),
        build_plan=build_plan,
        config_to_dict=lambda cfg: dict(TOY)))


# ------------------------------------------------- the plain implementation of it
def plain_forward(folder: str, tokens: List[int]) -> torch.Tensor:
    t = {k: v.float() for k, v in pm.read_safetensors(os.path.join(folder, "model.safetensors")).items()}
    T = len(tokens)
    residual = t["embed.weight"][torch.tensor(tokens)]
    cos, sin = pm.rope_table(T, 8, 1e4)
    norm = lambda x, name: pm.rms_norm(x, t[name], EPS, False)

    def moe(p, h):
        w, ids = pm.route(h, t[f"{p}.moe.router.weight"], None, K, "softmax", True, 1.0)
        gate_up = [torch.cat([t[f"{p}.moe.e{e}.gate.weight"], t[f"{p}.moe.e{e}.up.weight"]]) for e in range(E)]
        down = [t[f"{p}.moe.e{e}.down.weight"] for e in range(E)]
        return pm.experts(h, w, ids, gate_up, down, "silu", 0, 0, lambda z: z)

    def attention(p, h):
        q = pm.apply_rope((h @ t[f"{p}.attn.q.weight"].t()).view(T, NQ, D), cos, sin, 8)
        k = pm.apply_rope((h @ t[f"{p}.attn.k.weight"].t()).view(T, NKV, D), cos, sin, 8)
        v = (h @ t[f"{p}.attn.v.weight"].t()).view(T, NKV, D)
        return pm.causal_attention(q, k, v, D ** -0.5, None).reshape(T, NQ * D) @ t[f"{p}.attn.o.weight"].t()

    def latent(p, h):
        c = h @ t[f"{p}.lat.c.weight"].t()
        means = c.cumsum(0) / torch.arange(1, T + 1)[:, None]
        return means @ t[f"{p}.lat.o.weight"].t()

    # blocks.0: three norms
    h = norm(residual, "blocks.0.n1.weight")
    a = norm(attention("blocks.0", h), "blocks.0.n_post.weight")
    residual = residual + a
    x = moe("blocks.0", norm(residual, "blocks.0.n2.weight"))
    # blocks.1: one norm, no feed-forward
    residual = residual + x
    x = latent("blocks.1", norm(residual, "blocks.1.n1.weight"))
    # blocks.2: the usual arrangement around the latent mixer
    residual = residual + x
    a = latent("blocks.2", norm(residual, "blocks.2.n1.weight"))
    residual = residual + a
    x = moe("blocks.2", norm(residual, "blocks.2.n2.weight"))
    return norm(residual + x, "final_norm.weight") @ t["head.weight"].t()


# ------------------------------------------------------------------------- tests
def test_a_layer_must_list_what_its_block_arranges():
    """Not a GPU test: the model refuses a layer whose parts do not fit its block kind."""
    from freetoken_b200.config.model_plan import LayerSpec, PartSpec
    from freetoken_b200.models import Model
    arch = register_toy_blocks()
    plan = arch.build_plan(arch.read_config(TOY))
    Model(plan)                                             # as planned: fine
    norm = plan.layers[1].mixer_norm
    from dataclasses import replace
    wrong_norms = replace(plan, layers=(plan.layers[0], replace(plan.layers[1], feed_forward_norm=norm),
                                        plan.layers[2]))
    with pytest.raises(ValueError, match="arranges the norms"):
        Model(wrong_norms)
    no_ffn = replace(plan, layers=(plan.layers[0], plan.layers[1], replace(plan.layers[2], feed_forward=None)))
    with pytest.raises(ValueError, match="needs feed-forward"):
        Model(no_ffn)
    twice = LayerSpec("x", PartSpec("prenorm", {}), plan.layers[0].mixer, plan.layers[0].feed_forward, norm, norm,
                      norms={"mixer": norm})
    with pytest.raises(ValueError, match="given twice"):
        twice.all_norms()


@pytest.fixture(scope="module")
def toy_folder(tmp_path_factory):
    from freetoken_b200.models import Model
    from freetoken_b200.weights import RandomOptions, write_model_folder
    arch = register_toy_blocks()
    folder = str(tmp_path_factory.mktemp("toyblocks"))
    model = Model(arch.build_plan(arch.read_config(TOY)))
    write_model_folder(folder, TOY, model.tensor_specs(), 9, torch.float32, RandomOptions(matrix_std=0.1, norm_std=0.1))
    return folder


@pytest.mark.gpu
def test_groups_and_storage_follow_the_needs(toy_folder):
    from freetoken_b200.engine import Engine, EngineArgs
    engine = Engine.from_folder(toy_folder, EngineArgs(dtype="float32", page_size=4, max_tokens=64,
                                                       max_running_requests=2))
    kinds = [g.need.kind for g in engine.cache.paged_groups]
    assert kinds == ["paged_kv", "toy_latent"]
    assert [g.stops for g in engine.cache.paged_groups] == [[0], [1, 2]]     # the two latent stops share a group
    kv, lat = engine.storage.paged
    assert tuple(kv.shape) == (1, 2, 17, NKV, 4, D) and kv.dtype == torch.float32
    assert tuple(lat.shape) == (2, 17, 4, W) and lat.dtype == torch.float32
    assert len(engine.model.blocks[0].norms) == 3 and engine.model.blocks[1].feed_forward is None
    assert not engine._graphs_allowed               # the toy mixer does not say it can be captured


@pytest.mark.gpu
@pytest.mark.parametrize("cut", ["whole", "decode_tail", "portions", "mixed"])
def test_toy_blocks_step_like_their_plain_implementation(toy_folder, cut):
    from freetoken_b200.engine import Engine, EngineArgs
    reqs = {f"r{i}": tiny.tokens(60 + i, n, V) for i, n in enumerate([2, 23, 37, 11, 29])}
    fn = {"whole": rd.whole, "decode_tail": lambda r: rd.decode_tail(r, 9), "portions": rd.portions,
          "mixed": rd.mixed}[cut]
    schedule = fn(reqs)
    engine = Engine.from_folder(toy_folder, EngineArgs(dtype="float32", page_size=4,
                                                       num_pages=-(-rd.peak_tokens(schedule, 4) // 4),
                                                       max_running_requests=4, poison_freed_pages=True))
    got = rd.run_engine(engine, reqs, schedule)
    for rid, toks in reqs.items():
        want = plain_forward(toy_folder, toks)
        assert torch.allclose(got[rid], want, atol=5e-5, rtol=1e-4), (cut, rid, (got[rid] - want).abs().max())
    assert engine.cache.free_pages() == engine.cache.total_pages()
    # both groups' pages went back, and free pages of the latent group are poisoned too
    assert torch.isnan(engine.storage.paged[1][:, 1:]).all()
