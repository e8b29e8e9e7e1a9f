"""The tensor-core paths at the sizes they serve: the tcgen05 grouped GEMM with
many tiles per CTA (its persistent loop, both TMEM accumulator buffers, ring
parity carried across tiles) at K = 3072 / 1536, skewed expert loads included;
the engine at real layer width against the plain implementation; and the
attention kernels at contexts of tens of thousands of keys.

The reference's policy is the same - a kernel beside a plain loop at the
served shape (tests/moe/test_fused_moe.py:61-157,
tests/kernels/test_triton_attention.py:247-355).
"""

import pytest
import torch

import replay_driver as rd
import test_engine_gpu as eg
import tiny
from test_kernels_gpu import _glu

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
TOL = dict(atol=1e-2, rtol=1.6e-2)


def ops():
    from freetoken_b200.csrc import ops as o
    return o


def rnd(*shape, seed=0, scale=1.0, dtype=torch.bfloat16):
    g = torch.Generator(device=DEV).manual_seed(seed)
    return (torch.randn(*shape, generator=g, device=DEV) * scale).to(dtype)


# ------------------------------------------------------ grouped GEMM, many tiles
def _routes(counts, k, seed=0):
    """Sorted routes for the given rows per expert: route r belongs to token
    r // k; routes are dealt to experts in a shuffled order."""
    E = len(counts)
    R = sum(counts)
    assert R % k == 0
    g = torch.Generator().manual_seed(seed)
    flat = torch.repeat_interleave(torch.arange(E), torch.tensor(counts))[torch.randperm(R, generator=g)]
    order = torch.sort(flat, stable=True).indices.to(torch.int32)
    offsets = torch.zeros(E + 1, dtype=torch.int32)
    offsets[1:] = torch.tensor(counts).cumsum(0)
    return flat.to(DEV), order.to(DEV), (order // k).to(torch.int32).to(DEV), offsets.to(DEV)


def _even(E, R):
    return [R // E] * E


def _skewed(E, R):
    """One expert with a single row, one with 700, several empty, the rest uneven."""
    counts = [0] * E
    counts[3], counts[7] = 1, 700
    busy = [e for e in range(E) if e not in (3, 7, 0, 11, 12, 30)]
    left = R - 701
    for i, e in enumerate(busy):
        share = left // (len(busy) - i)
        share = max(1, share + (137 * (i % 5) - 274 if i < len(busy) - 1 else 0))
        counts[e] = min(share, left)
        left -= counts[e]
    counts[busy[-1]] += left
    assert sum(counts) == R and all(c >= 0 for c in counts)
    return counts


@pytest.mark.parametrize("load", ["even", "skewed"])
@pytest.mark.parametrize("act", ["silu", "swigluoai"])
def test_expert_gemms_tc_at_real_width(load, act):
    """32 experts of the real width (3072 -> 2 x 1536 -> 3072), 2,048 tokens top-8:
    1,500+ tiles of the gate_up product over at most 148 CTAs, so every CTA walks
    ten or more tiles, and 48 / 24 k-blocks per tile."""
    o = ops()
    from freetoken_b200.parts.base import Workspace
    E, k, T, H, I = 32, 8, 2048, 3072, 1536
    R = T * k
    counts = _even(E, R) if load == "even" else _skewed(E, R)
    flat, sorted_route, sorted_token, offsets = _routes(counts, k)
    x = rnd(T, H, seed=1)
    w1 = rnd(E, 2 * I, H, seed=2, scale=0.02)
    w2 = rnd(E, H, I, seed=3, scale=0.02)
    rw = torch.rand(R, generator=torch.Generator().manual_seed(4)).to(DEV)
    mid = torch.full((R, I), float("nan"), dtype=torch.bfloat16, device=DEV)
    parts = torch.full((R, H), float("nan"), dtype=torch.bfloat16, device=DEV)
    busy = (offsets[1:] > offsets[:-1]).nonzero().flatten().to(torch.int32)
    active = torch.cat([busy, torch.zeros(E - busy.numel(), dtype=torch.int32, device=DEV),
                        torch.tensor([busy.numel()], dtype=torch.int32, device=DEV)])
    ws = Workspace(DEV)
    o.moe_experts_tc(x, w1, w2, mid, parts, offsets, active, sorted_route, sorted_token, rw, R, act,
                     1.702, 7.0, ws)
    torch.cuda.synchronize()
    o.check_tc_status(DEV)
    inv = torch.empty(R, dtype=torch.long, device=DEV)
    inv[sorted_route.long()] = torch.arange(R, device=DEV)
    for e in range(E):
        rs = (flat == e).nonzero().flatten()
        if rs.numel() == 0:
            continue
        gu = x[rs // k].float() @ w1[e].float().t()
        m = _glu(gu[:, :I], gu[:, I:], act)
        got_mid = mid[inv[rs]].float()
        assert torch.allclose(got_mid, m, **TOL), (e, "mid", (got_mid - m).abs().max().item())
        y = (got_mid @ w2[e].float().t()) * rw[rs][:, None]
        got = parts[rs].float()
        assert torch.allclose(got, y, **TOL), (e, "down", (got - y).abs().max().item())


# --------------------------------------------- the engine at real layer width
def real_width_config():
    from freetoken_b200.benchmark import BENCH_CONFIG
    return dict(BENCH_CONFIG, num_hidden_layers=1, num_local_experts=16, num_experts_per_tok=4,
                vocab_size=4096, max_position_embeddings=1024)


@pytest.fixture(scope="module")
def real_width_folder(tmp_path_factory):
    """One layer of the real width (hidden 3072, 48/8 heads of 128, rotary 64,
    per-layer QK norm, expert width 1536) with 16 experts top-4 and a vocabulary
    of 4,096: about 0.6 GB."""
    from freetoken_b200.benchmark import bench_random_options
    from freetoken_b200.models import Model
    from freetoken_b200.registry import architecture_of
    from freetoken_b200.weights import write_model_folder
    folder = str(tmp_path_factory.mktemp("real_width"))
    cfg = real_width_config()
    arch = architecture_of(cfg)
    model = Model(arch.build_plan(arch.read_config(cfg)))
    write_model_folder(folder, cfg, model.tensor_specs(), 5, torch.bfloat16,
                       bench_random_options(router_bias_std=0.01))
    return folder


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_engine_at_real_width_matches_plain(real_width_folder, dtype, monkeypatch):
    """A 608-token prompt in one step (in bfloat16: the tcgen05 grouped GEMM and
    the tcgen05 attention, asserted) and 32 tokens decoded one by one, against
    the plain implementation's whole-sequence logits at every position."""
    o = ops()
    calls = {"moe_gemm_tc": 0, "attn_prefill_tc": 0, "attn_decode": 0, "skinny_gemm": 0}
    for name in calls:
        real = getattr(o, name)
        monkeypatch.setattr(o, name, (lambda real, name: lambda *a, **k: (
            calls.__setitem__(name, calls[name] + 1), real(*a, **k))[1])(real, name))
    cfg = real_width_config()
    toks = tiny.tokens(11, 640, cfg["vocab_size"])
    reqs = {"r": toks}
    schedule = rd.decode_tail(reqs, tail=32)
    engine = eg.make_engine(real_width_folder, dtype, 64, rd.peak_tokens(schedule, 64), live=1)
    models = {"R": real_width_folder}
    if dtype == "float32":
        got = rd.run_engine(engine, reqs, schedule)
        want = eg.plain_logits(models, "R", dtype, reqs)
        assert not any(calls.values())
    else:
        routing = {}
        got = rd.run_engine(engine, reqs, schedule, routing)
        o.check_tc_status(engine.device)
        want = eg.plain_logits(models, "R", dtype, reqs, routing)
        assert calls["moe_gemm_tc"] >= 2 and calls["attn_prefill_tc"] >= 1, calls
        assert calls["attn_decode"] >= 32 and calls["skinny_gemm"] >= 32, calls
    assert want["r"].abs().max() > 1.0, "logits too small for the comparison to mean anything"
    eg.compare(got, want, dtype, "real width, decode tail")
    assert engine.cache.free_pages() == engine.cache.total_pages()


# ------------------------------------------------------------- long contexts
def _long_case(nq, nkv, d, P, lens, seed, poison):
    """Segments (pos0, n) over shuffled pages; queries scaled so that a few keys
    anywhere in the context carry most of the weight (a wrong tile, split or page
    then changes the output by O(1)).  With ``poison`` every slot past a
    segment's last key is NaN."""
    S = len(lens)
    total = [p + n for p, n in lens]
    width = max(-(-t // P) for t in total)
    pages = S * width + 1
    g = torch.Generator(device=DEV).manual_seed(seed)
    table = (torch.randperm(pages - 1, generator=g, device=DEV)[: S * width] + 1).to(torch.int32).view(S, width)
    kv = torch.randn(2, pages, nkv, P, d, generator=g, device=DEV).to(torch.bfloat16)
    T = sum(n for _, n in lens)
    q = (torch.randn(T, nq * d, generator=g, device=DEV) * 4.0).to(torch.bfloat16)
    pos = torch.cat([torch.arange(p, p + n) for p, n in lens]).to(torch.int32).to(DEV)
    seg = torch.cat([torch.full((n,), s) for s, (_, n) in enumerate(lens)]).to(torch.int32).to(DEV)
    if poison:
        kv[:, 0] = float("nan")
        for s, t in enumerate(total):
            first = t // P
            if t % P:
                kv[:, int(table[s, first]), :, t % P:] = float("nan")
                first += 1
            if first < width:
                kv[:, table[s, first:].long()] = float("nan")
    return q, kv, pos, seg, table


def _long_ref(q, kv, lens, table, nq, nkv, d, P, scale):
    """Plain float32 attention on the device, one segment at a time."""
    G = nq // nkv
    out = torch.empty(q.shape, dtype=torch.float32, device=DEV)
    row = 0
    for s, (p0, n) in enumerate(lens):
        L = p0 + n
        pages = table[s, : -(-L // P)].long()
        K = kv[0, pages].permute(1, 0, 2, 3).reshape(nkv, -1, d)[:, :L].float()
        V = kv[1, pages].permute(1, 0, 2, 3).reshape(nkv, -1, d)[:, :L].float()
        qs = q[row: row + n].view(n, nkv, G, d).float()
        scores = torch.einsum("tkgd,kjd->kgtj", qs, K) * scale
        keys = torch.arange(L, device=DEV)[None, :]
        me = (p0 + torch.arange(n, device=DEV))[:, None]
        scores = scores.masked_fill(keys > me, float("-inf"))
        w = torch.softmax(scores, dim=-1)
        out[row: row + n] = torch.einsum("kgtj,kjd->tkgd", w, V).reshape(n, nq * d)
        row += n
    return out


@pytest.mark.parametrize("poison", [False, True])
@pytest.mark.parametrize("positions", [[32767 - 3 * i for i in range(8)], [65535 - 41], [65535]])
def test_attn_decode_long_context(positions, poison):
    """8 x 32K and 1 x 64K keys, 48 query heads over 8 KV heads of 128: dozens of
    splits, block-table rows of up to 1,024 pages, last pages partly filled."""
    from freetoken_b200.parts.base import Workspace
    o = ops()
    nq, nkv, d, P = 48, 8, 128, 64
    lens = [(p, 1) for p in positions]
    q, kv, pos, seg, table = _long_case(nq, nkv, d, P, lens, seed=len(positions), poison=poison)
    scale = d ** -0.5
    want = _long_ref(q, kv, lens, table, nq, nkv, d, P, scale)
    for tma in (True, False):
        out = torch.zeros_like(q)
        o.DECODE_TMA = tma
        try:
            o.attn_decode(q, out, kv, None, len(positions), pos, seg, table, nq, nkv, d, scale, None,
                          max(positions) + 1, Workspace(DEV))
        finally:
            o.DECODE_TMA = True
        o.check_tc_status(DEV)
        assert want.abs().max() > 0.5
        assert torch.allclose(out.float(), want, **TOL), (tma, (out.float() - want).abs().max().item())


@pytest.mark.parametrize("poison", [False, True])
@pytest.mark.parametrize("lens", [[(4096, 4096)], [(8000, 190), (0, 1500)]])
def test_attn_prefill_tc_long_context(lens, poison):
    """A 4,096-token portion on a 4,096-token prefix (128 key tiles per CTA at the
    end), and a short portion far into a context beside a fresh prompt."""
    o = ops()
    nq, nkv, d, P = 8, 2, 128, 64
    q, kv, pos, seg, table = _long_case(nq, nkv, d, P, lens, seed=7, poison=poison)
    scale = d ** -0.5
    want = _long_ref(q, kv, lens, table, nq, nkv, d, P, scale)
    out = torch.zeros_like(q)
    starts = [0]
    for _, n in lens:
        starts.append(starts[-1] + n)
    tiles = [(s, q0) for s, (_, n) in enumerate(lens) for q0 in range(0, n, 64)]
    dev = lambda xs: torch.tensor(xs, dtype=torch.int32, device=DEV)
    assert o.attn_prefill_tc_takes(q, kv, d, None)
    o.attn_prefill_tc(q, out, kv, dev([t[0] for t in tiles]), dev([t[1] for t in tiles]), dev(starts),
                      dev([p for p, _ in lens]), table, nq, nkv, d, scale)
    o.check_tc_status(DEV)
    assert want.abs().max() > 0.5
    assert torch.allclose(out.float(), want, **TOL), (out.float() - want).abs().max().item()


@pytest.mark.parametrize("n", [608, 2048])
def test_attn_prefill_tc_repeats_bitwise_on_a_full_grid(n):
    """48 query heads over 8 KV heads of 128: hundreds of CTAs, two per SM, whose
    softmax warps drift apart by more than a key tile when a V tile arrives late.
    The same launch thirty times must give the same bits, and the right ones (a
    warp that read its accumulator one product early used to show up here as 32
    wrong rows of one head, about once per launch)."""
    o = ops()
    nq, nkv, d, P = 48, 8, 128, 64
    lens = [(0, n)]
    q, kv, pos, seg, table = _long_case(nq, nkv, d, P, lens, seed=3, poison=False)
    scale = d ** -0.5
    tiles = [(0, q0) for q0 in range(0, n, 64)]
    dev = lambda xs: torch.tensor(xs, dtype=torch.int32, device=DEV)
    ts, tq, st, p0 = dev([t[0] for t in tiles]), dev([t[1] for t in tiles]), dev([0, n]), dev([0])
    outs = []
    for _ in range(30):
        out = torch.zeros_like(q)
        o.attn_prefill_tc(q, out, kv, ts, tq, st, p0, table, nq, nkv, d, scale)
        outs.append(out)
    torch.cuda.synchronize()
    o.check_tc_status(DEV)
    want = _long_ref(q, kv, lens, table, nq, nkv, d, P, scale)
    assert torch.allclose(outs[0].float(), want, **TOL), (outs[0].float() - want).abs().max().item()
    for i, out in enumerate(outs[1:], 1):
        assert torch.equal(out, outs[0]), f"launch {i} differs from launch 0"
