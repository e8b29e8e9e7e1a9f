"""Each part of a layer alone - norm, position encoding, mixer, feed-forward,
embedding and head - built from a PartSpec, given random tensors, run on a
hand-made step and compared with the plain implementation's function for it."""

import pytest
import torch

import plain_model as pm

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
TOL = {"float32": dict(atol=2e-5, rtol=1e-4), "bfloat16": dict(atol=2e-2, rtol=2e-2)}


def make_ctx(dtype, segments, page, tokens=None):
    """A StepContext for segments [(pos0, n), ...] with shuffled pages."""
    from freetoken_b200.parts import Segment, StepContext, Workspace
    segs, q = [], 0
    for slot, (p0, n) in enumerate(segments):
        segs.append(Segment(slot, p0, n, q))
        q += n
    T = q
    width = max(-(-(p0 + n) // page) for p0, n in segments)
    pages = len(segments) * width + 1
    table = (torch.randperm(pages - 1)[: len(segments) * width] + 1).to(torch.int32).view(len(segments), width)
    i32 = lambda xs: torch.tensor(xs, dtype=torch.int32, device=DEV)
    pos = [p for p0, n in segments for p in range(p0, p0 + n)]
    seg_of = [i for i, (_, n) in enumerate(segments) for _ in range(n)]
    ctx = StepContext(
        device=torch.device(DEV), dtype=DT[dtype], segments=segs, num_tokens=T,
        token_ids=i32(tokens if tokens is not None else [0] * T), token_pos=i32(pos), token_seg=i32(seg_of),
        seg_slot=i32([s.slot for s in segs]), seg_pos0=i32([s.pos0 for s in segs]),
        seg_q_start=i32([s.q_start for s in segs] + [T]), seg_kv_len=i32([s.pos0 + s.n for s in segs]),
        block_tables=[table.to(DEV)], workspace=Workspace(DEV), page_size=page,
        max_q_len=max(n for _, n in segments), max_kv_len=max(p0 + n for p0, n in segments),
        max_positions=256)          # a part that plans step metadata does so at its first use
    return ctx, pages


def random_tensors(part, dtype, seed=0):
    from freetoken_b200.weights import RandomOptions, random_state
    return random_state(part.tensor_specs(), seed, DEV, DT[dtype], torch.bfloat16,
                        RandomOptions(matrix_std=0.08, norm_std=0.2, router_bias_std=0.05))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("plus_one", [False, True])
def test_norm_part(dtype, plus_one):
    from freetoken_b200.config import PartSpec
    from freetoken_b200.parts import NORMS
    part = NORMS.get("rmsnorm")(PartSpec("rmsnorm", {"size": 80, "eps": 1e-5, "plus_one": plus_one, "scope": "ln"}), "m")
    t = random_tensors(part, dtype)
    assert list(t) == ["m.ln.weight"]
    part.bind(t, DT[dtype])
    ctx, _ = make_ctx(dtype, [(0, 5)], 4)
    delta = torch.randn(5, 80, device=DEV).to(DT[dtype])
    residual = torch.randn(5, 80, device=DEV)
    want_res = residual + delta.float()
    out = part.forward(ctx, delta, residual)
    assert torch.allclose(residual, want_res, atol=1e-6)
    assert torch.allclose(out.float(), pm.rms_norm(want_res.cpu(), t["m.ln.weight"].cpu(), 1e-5, plus_one).to(DEV), **TOL[dtype])


def test_position_parts():
    from freetoken_b200.config import PartSpec
    from freetoken_b200.parts import POSITIONS
    spec = PartSpec("rotary_neox", {"head_dim": 32, "rotary_dim": 12, "theta": 5e6, "max_position": 100})
    rope = POSITIONS.get("rotary_neox")(spec, "")
    table = rope.table(DEV, 64)
    cos, sin = pm.rope_table(64, 12, 5e6)
    assert table.shape == (64, 12) and torch.equal(table.cpu(), torch.cat([cos, sin], -1))
    assert rope.table(DEV, 1000).shape[0] == 100            # cut at max_position
    assert not rope.interleaved and POSITIONS.get("rotary_interleaved")(spec, "").interleaved
    none = POSITIONS.get("none")(PartSpec("none", {}), "")
    assert none.table(DEV, 10) is None and none.rotary_dim == 0
    with pytest.raises(ValueError):
        POSITIONS.get("rotary_neox")(PartSpec("rotary_neox", {**spec.params, "rotary_dim": 7}), "")


ATTN = dict(hidden_size=96, num_heads=6, num_kv_heads=2, head_dim=32, sm_scale=32 ** -0.5, qk_norm_eps=1e-6,
            qk_norm_plus_one=False, scope="attn",
            checkpoint_names={"qkv": "qkv.weight", "o": "o.weight", "q": "q.weight", "k": "k.weight",
                              "v": "v.weight", "q_norm": "qn.weight", "k_norm": "kn.weight"})


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("qk_norm,rotary,window", [("per_layer", 16, None), ("none", 32, 5), ("per_head", 0, None)])
def test_attention_part_whole_then_token_by_token(dtype, qk_norm, rotary, window):
    """The mixer alone: a 70-token prompt whole, then 6 tokens one by one, against
    the plain functions on the whole 76-token sequence."""
    from freetoken_b200.config import PartSpec
    from freetoken_b200.parts import MIXERS, CacheView
    pos_spec = PartSpec("rotary_neox" if rotary else "none",
                        {"head_dim": 32, "rotary_dim": rotary, "theta": 1e4, "max_position": 256})
    part = MIXERS.get("paged_attention")(PartSpec("paged_attention", {
        **ATTN, "qk_norm": qk_norm, "sliding_window": window, "position": pos_spec}), "L")
    t = random_tensors(part, dtype)
    part.bind(t, DT[dtype])
    need = part.cache_need()
    assert (need.num_kv_heads, need.head_dim, need.window) == (2, 32, window)
    T, page = 76, 8
    x = (torch.randn(T, 96, generator=torch.Generator().manual_seed(1))).to(DT[dtype]).to(DEV)
    ctx, pages = make_ctx(dtype, [(0, 70)], page)
    # one table for the whole life of the request: wide enough for 76 tokens
    width = -(-T // page)
    table = (torch.randperm(width) + 1).to(torch.int32).view(1, width).to(DEV)
    kv = torch.zeros(2, width + 1, 2, page, 32, dtype=DT[dtype], device=DEV)
    ctx.block_tables = [table]
    got = [part.forward(ctx, x[:70], CacheView(kv_pages=kv)).clone()]
    for i in range(70, T):
        step, _ = make_ctx(dtype, [(i, 1)], page)
        step.block_tables = [table]
        got.append(part.forward(step, x[i:i + 1], CacheView(kv_pages=kv)).clone())
    got = torch.cat(got).float().cpu()

    xf = x.float().cpu()
    w = {k: v.float().cpu() for k, v in t.items()}
    qkv = xf @ w["L.attn.qkv.weight"].t()
    q, k, v = qkv[:, :192], qkv[:, 192:256], qkv[:, 256:]
    q, k = pm.qk_norm(q, k, w.get("L.attn.qn.weight"), w.get("L.attn.kn.weight"), qk_norm, 1e-6, False, 6, 2, 32)
    cos, sin = pm.rope_table(T, rotary, 1e4) if rotary else (None, None)
    q = pm.apply_rope(q.view(T, 6, 32), cos, sin, rotary)
    k = pm.apply_rope(k.view(T, 2, 32), cos, sin, rotary)
    o = pm.causal_attention(q, k, v.reshape(T, 2, 32), 32 ** -0.5, window).reshape(T, 192)
    want = o @ w["L.attn.o.weight"].t()
    assert torch.allclose(got, want, **TOL[dtype]), (got - want).abs().max()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("scoring,use_bias,renorm,scale,act,T", [
    ("sigmoid", True, True, 2.0, "silu", 7), ("softmax", False, False, 1.0, "swigluoai", 150)])
def test_routed_experts_part(dtype, scoring, use_bias, renorm, scale, act, T):
    from freetoken_b200.config import PartSpec
    from freetoken_b200.parts import FEED_FORWARDS
    E, k, H, I = 8, 3, 64, 40
    part = FEED_FORWARDS.get("routed_experts")(PartSpec("routed_experts", {
        "hidden_size": H, "intermediate_size": I, "num_experts": E, "top_k": k, "scoring": scoring,
        "use_bias": use_bias, "renormalize": renorm, "scale": scale, "activation": act,
        "act_alpha": 1.702, "act_limit": 7.0, "scope": "moe",
        "checkpoint_names": {"router": "gate.weight", "bias": "bias", "gate_up": "gate_up", "down": "down",
                             "gate": "e{e}.w1", "up": "e{e}.w3", "down_each": "e{e}.w2"}}), "L")
    t = random_tensors(part, dtype)
    part.bind(t, DT[dtype])
    x = torch.randn(T, H, generator=torch.Generator().manual_seed(2)).to(DT[dtype]).to(DEV)
    ctx, _ = make_ctx(dtype, [(0, T)], 16)
    y = part.forward(ctx, x)
    assert y.shape == (T, k, H)                              # k partial rows per token for the next norm
    got = y.float().sum(1).cpu()
    ids, _ = part.route(ctx, x)
    w = {n: v.float().cpu() for n, v in t.items()}
    bias = w["L.moe.bias"] if use_bias else None
    wts, own = pm.route(x.float().cpu(), w["L.moe.gate.weight"], bias, k, scoring, renorm, scale,
                        forced_ids=ids.cpu())
    if dtype == "float32":
        _, free = pm.route(x.float().cpu(), w["L.moe.gate.weight"], bias, k, scoring, renorm, scale)
        assert torch.equal(free, ids.cpu().long())           # float32: the same experts, in the same order
    gate_up = [w["L.moe.gate_up"][e] for e in range(E)]
    down = [w["L.moe.down"][e] for e in range(E)]
    rnd = (lambda z: z.to(torch.bfloat16).float()) if dtype == "bfloat16" else (lambda z: z)
    want = pm.experts(x.float().cpu(), wts, own, gate_up, down, act, 1.702, 7.0, rnd)
    assert torch.allclose(got, want, **TOL[dtype]), (got - want).abs().max()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_embedding_and_head_parts(dtype):
    from freetoken_b200.config import PartSpec
    from freetoken_b200.parts import EMBEDDINGS, HEADS
    V, H = 300, 72
    emb = EMBEDDINGS.get("token_embedding")(PartSpec("token_embedding", {"vocab_size": V, "hidden_size": H, "scope": "embed"}), "m")
    t = random_tensors(emb, dtype)
    emb.bind(t, DT[dtype])
    ids = [5, 299, 0, 5]
    ctx, _ = make_ctx(dtype, [(0, 4)], 4, tokens=ids)
    residual = torch.empty(4, H, device=DEV)
    emb.forward(ctx, residual)
    assert torch.equal(residual, t["m.embed.weight"].float()[ids])
    for tied in (None, "m.embed.weight"):
        head = HEADS.get("lm_head")(PartSpec("lm_head", {"vocab_size": V, "hidden_size": H, "scope": "head", "tied_to": tied}), "")
        assert all(s.optional for s in head.tensor_specs()) == bool(tied)
        ht = dict(t) if tied else random_tensors(head, dtype, seed=3)
        head.bind(ht, DT[dtype])
        x = torch.randn(4, H, device=DEV).to(DT[dtype])
        out = torch.empty(4, V, device=DEV)
        head.forward(ctx, x, out)
        wname = tied or "head.weight"
        assert torch.allclose(out, x.float() @ ht[wname].float().t(), **TOL[dtype])
