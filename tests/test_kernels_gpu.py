"""Each CUDA kernel alone against a plain PyTorch float32 reference of the same
op, at sizes other than the engine's tiny models (odd widths, head sizes that
are no power of two, groups of 1/3/6, vocabularies like 1000)."""


import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
TOL = {"float32": dict(atol=1e-5, rtol=1e-5), "bfloat16": dict(atol=1e-2, rtol=1.6e-2)}


def ops():
    from freetoken_b200.csrc import ops as o
    return o


def rnd(*shape, dtype=torch.float32, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype).to(DEV)


# ------------------------------------------------------------- rows
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,vocab", [(40, 11), (3072, 100)])
def test_embed_gather(dtype, H, vocab):
    table = rnd(vocab, H, dtype=DT[dtype])
    ids = torch.tensor([3, 0, vocab - 1, 3, 7], dtype=torch.int32, device=DEV)
    out = torch.empty(5, H, dtype=torch.float32, device=DEV)
    ops().embed_gather(ids, table, out)
    assert torch.equal(out, table[ids.long()].float())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,plus_one,eps", [(96, False, 1e-5), (1000, True, 1e-6), (3072, False, 1e-6)])
def test_rmsnorm_residual(dtype, H, plus_one, eps):
    T = 7
    delta = rnd(T, H, dtype=DT[dtype], seed=1)
    res = rnd(T, H, seed=2)
    w = rnd(H, seed=3, scale=0.3) + (0.0 if plus_one else 1.0)
    res_in = res.clone()
    out = torch.empty(T, H, dtype=DT[dtype], device=DEV)
    ops().rmsnorm(delta, res, w, out, eps, plus_one)
    z = res_in + delta.float()
    want = z * torch.rsqrt(z.pow(2).mean(-1, keepdim=True) + eps) * (w + (1.0 if plus_one else 0.0))
    assert torch.allclose(res, z, atol=1e-6)
    assert torch.allclose(out.float(), want, **TOL[dtype])
    # without delta the residual is left alone
    res2 = res_in.clone()
    ops().rmsnorm(None, res2, w, out, eps, plus_one)
    assert torch.equal(res2, res_in)
    # k partial rows per token are summed in order
    parts = rnd(T, 3, H, dtype=DT[dtype], seed=9)
    res3 = res_in.clone()
    ops().rmsnorm(parts, res3, w, out, eps, plus_one)
    z3 = res_in + parts.float().sum(1)
    want3 = z3 * torch.rsqrt(z3.pow(2).mean(-1, keepdim=True) + eps) * (w + (1.0 if plus_one else 0.0))
    assert torch.allclose(res3, z3, atol=1e-5)
    assert torch.allclose(out.float(), want3, **TOL[dtype])


def _rope_ref(x, pos, R, theta, interleaved):
    if R == 0:
        return x
    inv = 1.0 / (theta ** (torch.arange(0, R, 2, dtype=torch.float) / R))
    f = pos.float()[:, None].cpu() * inv[None, :]
    c, s = f.cos().to(x.device)[:, None, :], f.sin().to(x.device)[:, None, :]
    y = x.clone()
    if interleaved:
        x0, x1 = x[..., 0:R:2], x[..., 1:R:2]
        y[..., 0:R:2] = x0 * c - x1 * s
        y[..., 1:R:2] = x1 * c + x0 * s
    else:
        h = R // 2
        x0, x1 = x[..., :h], x[..., h:R]
        y[..., :h] = x0 * c - x1 * s
        y[..., h:R] = x1 * c + x0 * s
    return y


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("nq,nkv,d,R,mode,interleaved,P", [
    (4, 2, 16, 8, 1, False, 4), (6, 3, 24, 24, 0, False, 8), (12, 2, 32, 16, 2, True, 16),
    (5, 5, 48, 0, 2, False, 2), (48, 8, 128, 64, 1, False, 64), (12, 4, 64, 32, 2, False, 16),
    (8, 2, 32, 32, 0, False, 8), (6, 2, 40, 16, 1, False, 8)])
def test_qk_rope_store(dtype, nq, nkv, d, R, mode, interleaved, P):
    o = ops()
    T, S, theta, eps = 9, 2, 12345.0, 1e-5
    qkv = rnd(T, (nq + 2 * nkv) * d, dtype=DT[dtype], seed=4)
    # two segments: positions 5.. (5 tokens) and 30.. (4 tokens)
    pos = torch.tensor([5, 6, 7, 8, 9, 30, 31, 32, 33], dtype=torch.int32, device=DEV)
    seg = torch.tensor([0] * 5 + [1] * 4, dtype=torch.int32, device=DEV)
    width = 40 // P + 1
    pages = S * width + 1
    table = (torch.randperm(pages - 1)[: S * width] + 1).to(torch.int32).view(S, width).to(DEV)
    kv = torch.zeros(2, pages, nkv, P, d, dtype=DT[dtype], device=DEV)
    qw = rnd(nq * d if mode == 1 else d, seed=5, scale=0.2) + 1.0
    kw = rnd(nkv * d if mode == 1 else d, seed=6, scale=0.2) + 1.0
    inv = 1.0 / (theta ** (torch.arange(0, max(R, 2), 2, dtype=torch.float) / max(R, 2)))
    tpos = torch.arange(64, dtype=torch.float)
    fr = torch.einsum("i,j->ij", tpos, inv)
    cos_sin = torch.cat((fr.cos(), fr.sin()), -1).to(DEV) if R else None
    q_out = torch.empty(T, nq * d, dtype=DT[dtype], device=DEV)
    o.qk_rope_store(qkv, q_out, kv, qw if mode else None, kw if mode else None, cos_sin, pos, seg,
                    table, nq, nkv, d, R, mode, False, interleaved, eps)
    x = qkv.float()
    q, k, v = x[:, :nq * d], x[:, nq * d:(nq + nkv) * d], x[:, (nq + nkv) * d:]

    def norm(z, w, heads):
        if mode == 0:
            return z
        if mode == 1:
            return z * torch.rsqrt(z.pow(2).mean(-1, keepdim=True) + eps) * w
        zh = z.view(T, heads, d)
        return (zh * torch.rsqrt(zh.pow(2).mean(-1, keepdim=True) + eps) * w).reshape(T, heads * d)

    qr = _rope_ref(norm(q, qw, nq).view(T, nq, d), pos, R, theta, interleaved).reshape(T, nq * d)
    kr = _rope_ref(norm(k, kw, nkv).view(T, nkv, d), pos, R, theta, interleaved)
    assert torch.allclose(q_out.float(), qr, **TOL[dtype])
    for t in range(T):
        page = int(table[int(seg[t]), int(pos[t]) // P])
        slot = int(pos[t]) % P
        assert torch.allclose(kv[0, page, :, slot].float(), kr[t], **TOL[dtype])
        assert torch.equal(kv[1, page, :, slot].float(), v[t].view(nkv, d))
    # a stop that reads another stop's cache writes nothing
    kv2 = torch.zeros_like(kv)
    o.qk_rope_store(qkv, q_out, None, qw if mode else None, kw if mode else None, cos_sin, pos, seg,
                    table, nq, nkv, d, R, mode, False, interleaved, eps)
    assert not kv2.any()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_combine(dtype):
    T, k, H = 5, 3, 100
    parts = rnd(T * k, H, dtype=DT[dtype])
    out = torch.empty(T, H, dtype=DT[dtype], device=DEV)
    ops().combine(parts, out, k)
    want = parts.float().view(T, k, H).sum(1)
    assert torch.allclose(out.float(), want, **TOL[dtype])


# ------------------------------------------------------------------ gemm
def _glu(g, u, act, alpha=1.702, limit=7.0):
    if act == "silu":
        return torch.nn.functional.silu(g) * u
    g = g.clamp(max=limit)
    u = u.clamp(-limit, limit)
    return g * torch.sigmoid(alpha * g) * (u + 1)


GEMM_TYPES = [("float32", "float32", "float32"), ("float32", "bfloat16", "float32"),
              ("bfloat16", "bfloat16", "bfloat16"), ("bfloat16", "bfloat16", "float32"),
              ("bfloat16", "float32", "float32")]


@pytest.mark.parametrize("at,wt,ct", GEMM_TYPES)
@pytest.mark.parametrize("M,N,K", [(1, 7, 5), (9, 100, 96), (70, 130, 257), (200, 130, 96)])
def test_gemm_rows_dense(at, wt, ct, M, N, K):
    a = rnd(M, K, dtype=DT[at], seed=1)
    w = rnd(N, K, dtype=DT[wt], seed=2, scale=0.1)
    c = torch.empty(M, N, dtype=DT[ct], device=DEV)
    ops().gemm_rows(a, w, c)
    want = a.float() @ w.float().t()
    tol = TOL["bfloat16" if ct == "bfloat16" else "float32"]
    assert torch.allclose(c.float(), want, atol=tol["atol"] * 3, rtol=tol["rtol"])
    if M >= 64 and K % 32 == 0:
        # many rows take the tiled kernel, few rows the simple one: the same bits
        few = torch.empty(8, N, dtype=DT[ct], device=DEV)
        ops().gemm_rows(a[100:108], w, few)
        assert torch.equal(few, c[100:108])


def _grouped_case(E, k, T, seed=0):
    g = torch.Generator().manual_seed(seed)
    ids = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(T)]).to(torch.int32)
    flat = ids.view(-1)
    order = torch.sort(flat.long(), stable=True).indices.to(torch.int32)
    counts = torch.bincount(flat.long(), minlength=E)
    offsets = torch.zeros(E + 1, dtype=torch.int32)
    offsets[1:] = counts.cumsum(0)
    return ids.to(DEV), order.to(DEV), (order // k).to(torch.int32).to(DEV), offsets.to(DEV)


@pytest.mark.parametrize("kernel", ["simt_f32", "simt_bf16", "skinny", "tc", "tc_weight_major", "tc_token_major"])
@pytest.mark.parametrize("E,k,T,H,I,act", [(4, 2, 5, 64, 32, "silu"), (8, 3, 19, 96, 48, "swigluoai"),
                                           (4, 2, 400, 96, 144, "swigluoai"),  # 200 rows per expert
                                           (16, 4, 150, 128, 80, "silu"), (3, 1, 40, 40, 24, "silu"),
                                           (8, 2, 700, 264, 200, "silu"),
                                           (4, 2, 650, 136, 72, "silu"),      # 325 rows per expert: three tiles each
                                           (1, 1, 300, 128, 80, "silu")])     # a single expert: still a 3-D weight map
def test_expert_gemms(kernel, E, k, T, H, I, act, monkeypatch):
    """gate_up + GLU, then down with the route weight, against a per-route loop."""
    o = ops()
    if kernel.startswith("tc_"):         # force one form of the GLU tile whatever the load
        monkeypatch.setattr(o, "TC_GLU_TOKEN_MAJOR_FROM_ROWS", 0 if kernel == "tc_token_major" else 1 << 30)
        kernel = "tc"
    dt = torch.float32 if kernel == "simt_f32" else torch.bfloat16
    x = rnd(T, H, dtype=dt, seed=1)
    w1 = rnd(E, 2 * I, H, dtype=dt, seed=2, scale=0.1)
    w2 = rnd(E, H, I, dtype=dt, seed=3, scale=0.1)
    ids, sorted_route, sorted_token, offsets = _grouped_case(E, k, T)
    rw = torch.rand(T * k, generator=torch.Generator().manual_seed(4)).to(DEV)
    R = T * k
    mid = torch.zeros(R, I, dtype=dt, device=DEV)
    parts = torch.zeros(R, H, dtype=dt, device=DEV)
    busy = (offsets[1:] > offsets[:-1]).nonzero().flatten().to(torch.int32)
    active = torch.cat([busy, torch.zeros(E - busy.numel(), dtype=torch.int32, device=DEV),
                        torch.tensor([busy.numel()], dtype=torch.int32, device=DEV)])
    if kernel == "tc":
        from freetoken_b200.parts.base import Workspace
        # few rows per expert: the weights are the M operand, gate and up two accumulators;
        # many: the tokens are the M operand, gate and up rows one N operand of 256
        o.moe_experts_tc(x, w1, w2, mid, parts, offsets, active, sorted_route, sorted_token, rw, R, act,
                         1.702, 7.0, Workspace(DEV))
        torch.cuda.synchronize()
        o.check_tc_status(DEV)
    elif kernel == "skinny":
        per = o.pass_rows(-(-R // E))
        o.skinny_gemm(x, w1, mid, group_offsets=offsets, active=active, a_rows=sorted_token,
                      rows=R, glu=True, act=act, rows_per_pass=per)
        o.skinny_gemm(mid, w2, parts, group_offsets=offsets, c_rows=sorted_route, row_scale=rw,
                      rows=R, rows_per_pass=per)
    else:
        o.gemm_rows(x, w1, mid, group_offsets=offsets, a_rows=sorted_token, rows=R, glu=True, act=act)
        o.gemm_rows(mid, w2, parts, group_offsets=offsets, c_rows=sorted_route, row_scale=rw, rows=R)
    tol = TOL["float32" if kernel == "simt_f32" else "bfloat16"]
    flat = ids.view(-1).long()
    # per-route reference, vectorised per expert
    inv = torch.empty(R, dtype=torch.long, device=DEV)
    inv[sorted_route.long()] = torch.arange(R, device=DEV)
    for e in range(E):
        rs = (flat == e).nonzero().flatten()
        if rs.numel() == 0:
            continue
        gu = x[rs // k].float() @ w1[e].float().t()
        m = _glu(gu[:, :I], gu[:, I:], act)
        got_mid = mid[inv[rs]].float()
        assert torch.allclose(got_mid, m, atol=tol["atol"], rtol=tol["rtol"]), (e, "mid")
        y = (got_mid @ w2[e].float().t()) * rw[rs][:, None]
        assert torch.allclose(parts[rs].float(), y, atol=tol["atol"], rtol=tol["rtol"]), (e, "down")


def test_moe_tile_map_covers_every_row_once_with_even_tiles():
    """The tile list of the tcgen05 grouped GEMM: per busy expert the fewest tiles of at
    most 128 rows, of equal size (in steps of 16), in expert order; empty entries after."""
    from freetoken_b200.parts.base import Workspace
    o = ops()
    counts = [0, 1, 700, 0, 128, 129, 260, 16, 0, 300]
    E = len(counts)
    offsets = torch.tensor([0] + list(torch.tensor(counts).cumsum(0)), dtype=torch.int32, device=DEV)
    busy = [e for e, c in enumerate(counts) if c]
    active = torch.tensor(busy + [0] * (E - len(busy)) + [len(busy)], dtype=torch.int32, device=DEV)
    rows = sum(counts)
    info = o.moe_tile_map(offsets, active, rows, E, Workspace(DEV)).cpu().tolist()
    want = []
    for e in busy:
        r, begin = counts[e], int(offsets[e])
        tiles = -(-r // 128)
        size = 128 if tiles == 1 else min(128, -(-(-(-r // tiles)) // 16) * 16)
        for i in range(tiles):
            row0 = begin + i * size
            left = begin + r - row0
            want.append([e, row0, min(size, -(-left // 16) * 16), begin + r])
    assert info[:len(want)] == want
    assert all(entry[0] == -1 for entry in info[len(want):])
    covered = sorted(row for e, row0, n, end in want for row in range(row0, min(row0 + n, end)))
    assert covered == list(range(rows))


@pytest.mark.parametrize("ct", ["bfloat16", "float32"])
@pytest.mark.parametrize("M,N,K", [(1, 40, 48), (8, 100, 96), (13, 1000, 264), (40, 64, 3072), (70, 33, 128)])
def test_skinny_gemm_dense(ct, M, N, K):
    o = ops()
    a = rnd(M, K, dtype=torch.bfloat16, seed=1)
    w = rnd(N, K, dtype=torch.bfloat16, seed=2, scale=0.1)
    c = torch.empty(M, N, dtype=DT[ct], device=DEV)
    o.skinny_gemm(a, w, c, rows_per_pass=o.pass_rows(M))
    want = a.float() @ w.float().t()
    tol = TOL[ct]
    assert torch.allclose(c.float(), want, atol=tol["atol"] * 3, rtol=tol["rtol"])


def test_skinny_gemm_refuses_odd_k():
    o = ops()
    a = rnd(2, 20, dtype=torch.bfloat16)
    w = rnd(8, 20, dtype=torch.bfloat16)
    c = torch.empty(2, 8, dtype=torch.bfloat16, device=DEV)
    assert not o.skinny_gemm_takes(a, w, c)
    with pytest.raises(o.KernelError):
        o.skinny_gemm(a, w, c)


# --------------------------------------------------------------- attention
def _paged_case(dtype, nq, nkv, d, P, lens, window=None, seed=0, standout=None):
    """Segments given as (pos0, n); K/V for positions < pos0+n live in shuffled pages."""
    S = len(lens)
    total = [p + n for p, n in lens]
    width = max(-(-t // P) for t in total)
    pages = S * width + 1
    g = torch.Generator().manual_seed(seed)
    table = (torch.randperm(pages - 1, generator=g)[: S * width] + 1).to(torch.int32).view(S, width)
    kv = torch.randn(2, pages, nkv, P, d, generator=g).to(DT[dtype])
    T = sum(n for _, n in lens)
    q = torch.randn(T, nq * d, generator=g).to(DT[dtype])
    pos, seg = [], []
    for s, (p0, n) in enumerate(lens):
        pos += list(range(p0, p0 + n))
        seg += [s] * n
    if standout is not None:
        # one far key that must win: scale one query and that key
        s_idx, key_pos = standout
        page = int(table[s_idx, key_pos // P])
        kv[0, page, :, key_pos % P] *= 6.0
    return (q.to(DEV), kv.to(DEV), torch.tensor(pos, dtype=torch.int32, device=DEV),
            torch.tensor(seg, dtype=torch.int32, device=DEV), table.to(DEV))


def _attn_ref(q, kv, pos, seg, table, nq, nkv, d, P, scale, window):
    T = q.shape[0]
    out = torch.zeros(T, nq, d)
    qf, kvf = q.float().cpu().view(T, nq, d), kv.float().cpu()
    for t in range(T):
        p, s = int(pos[t]), int(seg[t])
        lo = max(0, p - window + 1) if window else 0
        js = list(range(lo, p + 1))
        pages = [int(table[s, j // P]) for j in js]
        slots = [j % P for j in js]
        for h in range(nq):
            kh = h // (nq // nkv)
            K = torch.stack([kvf[0, pg, kh, sl] for pg, sl in zip(pages, slots)])
            V = torch.stack([kvf[1, pg, kh, sl] for pg, sl in zip(pages, slots)])
            w = torch.softmax((K @ qf[t, h]) * scale, 0)
            out[t, h] = w @ V
    return out.view(T, nq * d)


ATTN_CASES = [
    # nq, nkv, d, P, segments (pos0, n), window, standout
    (4, 2, 16, 4, [(0, 9)], None, None),
    (6, 1, 24, 8, [(0, 3), (17, 2), (40, 1)], None, None),
    (6, 6, 40, 16, [(31, 2), (64, 1)], None, (1, 2)),          # far key stands out
    (12, 2, 32, 16, [(0, 50), (200, 1)], None, (1, 33)),       # far key among hundreds
    (4, 2, 16, 4, [(0, 20), (37, 1)], 6, None),                # window edge inside pages
    (3, 1, 128, 64, [(120, 9), (1, 1)], 64, None),
]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("nq,nkv,d,P,lens,window,standout", ATTN_CASES)
def test_attn_paged_simt(dtype, nq, nkv, d, P, lens, window, standout):
    q, kv, pos, seg, table = _paged_case(dtype, nq, nkv, d, P, lens, window, standout=standout)
    out = torch.empty_like(q)
    scale = d ** -0.5
    ops().attn_paged_simt(q, out, kv, pos, seg, table, nq, nkv, d, scale, window)
    want = _attn_ref(q, kv, pos, seg, table, nq, nkv, d, P, scale, window)
    assert torch.allclose(out.float().cpu(), want, **TOL[dtype])


# ------------------------------------------------------------------ router
@pytest.mark.parametrize("E,k,softmax,renorm,use_bias,scale", [
    (4, 2, False, True, True, 1.0), (8, 3, True, False, False, 1.5), (256, 8, False, True, True, 2.0),
    (37, 5, True, True, False, 1.0), (5, 5, False, True, True, 1.0),
    (64, 40, False, True, True, 1.0), (100, 33, True, False, False, 2.0)])       # more choices than a warp has lanes
def test_router_select(E, k, softmax, renorm, use_bias, scale):
    T = 33
    logits = rnd(T, E, seed=1)
    logits[0, :] = 0.25          # all scores tie: lowest ids win
    bias = rnd(E, seed=2, scale=0.1) if use_bias else None
    if bias is not None:
        bias_row0 = bias.clone()
    ids = torch.empty(T, k, dtype=torch.int32, device=DEV)
    w = torch.empty(T, k, dtype=torch.float32, device=DEV)
    ops().router_select(logits, bias, ids, w, k, softmax, renorm, scale)
    s = torch.softmax(logits, -1) if softmax else torch.sigmoid(logits)
    c = s + (bias if bias is not None else 0)
    for t in range(T):
        order = sorted(range(E), key=lambda e: (-float(c[t, e]), e))[:k]
        assert ids[t].tolist() == order, t
    want = s.gather(1, ids.long())
    if renorm:
        want = want / (want.sum(-1, keepdim=True) + 1e-20)
    assert torch.allclose(w, want * scale, atol=1e-6, rtol=1e-5)
    if bias is None:
        assert ids[0].tolist() == list(range(k))


@pytest.mark.parametrize("T,E,k,softmax,renorm,use_bias,scale,terms", [
    (1, 256, 8, False, True, True, 2.0, 1), (8, 256, 8, False, True, True, 1.0, 1),
    (7, 37, 5, True, False, False, 1.5, 1), (3, 5, 5, False, True, False, 0.5, 1),
    (7, 600, 32, True, True, True, 1.0, 1), (8, 48, 4, False, True, True, 1.0, 3)])
def test_route_small_equals_select_then_sort(T, E, k, softmax, renorm, use_bias, scale, terms):
    """One launch for a handful of tokens: the same ids, weights, counts, offsets,
    sorted routes and busy-expert list as router_select followed by moe_sort."""
    o = ops()
    logits = rnd(T, E * terms, seed=5)
    logits[0, :] = 0.25
    bias = rnd(E, seed=6, scale=0.1) if use_bias else None
    R = T * k
    i32 = lambda n, fill=-1: torch.full((n,), fill, dtype=torch.int32, device=DEV)

    def buffers():
        return dict(ids=i32(R).view(T, k), w=torch.zeros(T, k, device=DEV), counts=i32(E),
                    offsets=i32(E + 1), sr=i32(R), st=i32(R), active=i32(E + 1))
    a, b = buffers(), buffers()
    o.router_select(logits, bias, a["ids"], a["w"], k, softmax, renorm, scale, terms)
    o.moe_sort(a["ids"].view(-1), a["counts"], a["offsets"], a["sr"], a["st"], a["active"], E, k)
    assert o.route_small_takes(T, E, k)
    o.route_small(logits, bias, b["ids"], b["w"], b["counts"], b["offsets"], b["sr"], b["st"], b["active"],
                  k, softmax, renorm, scale, terms)
    busy = int(a["active"][E])
    for name in ("ids", "counts", "offsets", "sr", "st"):
        assert torch.equal(a[name], b[name]), name
    assert torch.equal(a["w"], b["w"])
    assert int(b["active"][E]) == busy and torch.equal(a["active"][:busy], b["active"][:busy])


@pytest.mark.parametrize("T,E,H", [(70, 6, 128), (300, 256, 3072), (129, 37, 200)])
def test_router_logits_from_bf16_terms(T, E, H):
    """The float32 router weight split into three bfloat16 terms: the terms sum
    to the weight exactly, and tensor-core products of bfloat16 activations with
    them, summed by the selection kernel, give the float32 logits."""
    from freetoken_b200.parts import linear
    from freetoken_b200.parts.moe import bf16_terms
    x = rnd(T, H, dtype=torch.bfloat16, seed=1)
    w = rnd(E, H, seed=2, scale=0.05)
    terms = bf16_terms(w)
    assert terms.shape == (3 * E, H) and terms.dtype == torch.bfloat16
    assert torch.equal(terms.float().view(3, E, H).sum(0), w)
    parts = torch.empty(T, 3 * E, device=DEV)
    if not linear.library_f32_out(x, terms, parts):
        pytest.skip("this PyTorch has no bfloat16 product with a float32 result")
    want = x.double() @ w.double().t()
    got = parts.view(T, 3, E).sum(1)
    assert torch.allclose(got.double(), want, atol=2e-5, rtol=1e-5)
    # the selection sums the terms itself
    k = min(4, E)
    ids = torch.empty(T, k, dtype=torch.int32, device=DEV)
    wts = torch.empty(T, k, device=DEV)
    ops().router_select(parts, None, ids, wts, k, False, True, 1.0, terms=3)
    ids2 = torch.empty_like(ids)
    wts2 = torch.empty_like(wts)
    ops().router_select(got.contiguous(), None, ids2, wts2, k, False, True, 1.0)
    assert torch.equal(ids, ids2) and torch.allclose(wts, wts2, atol=1e-6)


@pytest.mark.parametrize("chunked", [False, True])
@pytest.mark.parametrize("E,k,T", [(4, 2, 1), (8, 3, 50), (256, 8, 300), (5, 1, 64), (37, 5, 1111),
                                   (1500, 2, 700)])
def test_moe_sort_is_stable_counting_sort(E, k, T, chunked):
    ids, want_route, want_token, want_off = _grouped_case(E, k, T, seed=3)
    R = T * k
    scratch = None
    if chunked:
        scratch = torch.full((ops().moe_sort_scratch(R, E),), -7, dtype=torch.int32, device=DEV)
    counts = torch.empty(E, dtype=torch.int32, device=DEV)
    offsets = torch.empty(E + 1, dtype=torch.int32, device=DEV)
    sr = torch.empty(R, dtype=torch.int32, device=DEV)
    st = torch.empty(R, dtype=torch.int32, device=DEV)
    active = torch.full((E + 1,), -1, dtype=torch.int32, device=DEV)
    ops().moe_sort(ids.view(-1), counts, offsets, sr, st, active, E, k, scratch)
    busy = (want_off[1:] > want_off[:-1]).nonzero().flatten().to(torch.int32)
    assert int(active[E]) == busy.numel()
    assert torch.equal(active[:busy.numel()], busy)
    assert torch.equal(offsets, want_off)
    assert torch.equal(sr, want_route)
    assert torch.equal(st, want_token)


# ---------------------------------------------------------------- sampling
def _sample_ref(logits, T, top_k, top_p, u):
    p = torch.exp((logits - logits.max()) / T).double()
    keep = torch.ones_like(p, dtype=torch.bool)
    if 0 < top_k < p.numel():
        kth = torch.sort(p, descending=True).values[top_k - 1]
        keep &= p >= kth
    if top_p < 1.0:
        srt = torch.sort(torch.where(keep, p, torch.zeros_like(p)), descending=True).values
        mass = srt.cumsum(0)
        cut = srt[int((mass >= top_p * srt.sum()).nonzero()[0])]
        keep &= p >= cut
    kept = torch.where(keep, p, torch.zeros_like(p))
    cdf = kept.cumsum(0)
    target = u * cdf[-1]
    return int((cdf > target).nonzero()[0]), cdf, target


@pytest.mark.parametrize("V", [50, 1000, 200064])
def test_sample(V):
    rows = 6
    logits = rnd(rows, V, seed=5, scale=2.0)
    temps = torch.tensor([0.0, 0.8, 1.0, 0.5, 1.3, 0.7], device=DEV)
    top_k = torch.tensor([0, 0, 5, 0, 40, 1], dtype=torch.int32, device=DEV)
    top_p = torch.tensor([1.0, 1.0, 1.0, 0.6, 0.9, 1.0], device=DEV)
    u = torch.tensor([0.3, 0.77, 0.12, 0.5, 0.93, 0.4], device=DEV)
    out = torch.empty(rows, dtype=torch.int32, device=DEV)
    probs = torch.empty(rows * V, device=DEV)
    ops().sample(logits, temps, top_k, top_p, u, out, probs)
    got = out.tolist()
    assert got[0] == int(logits[0].argmax())
    assert got[5] == int(logits[5].argmax())          # top_k = 1 is greedy
    lc = logits.cpu()
    for r in range(1, 5):
        want, cdf, target = _sample_ref(lc[r], float(temps[r]), int(top_k[r]), float(top_p[r]), float(u[r]))
        if got[r] != want:
            # float32 vs float64 running sums may differ right at a boundary
            assert abs(float(cdf[got[r]] - target)) < 1e-4 * float(cdf[-1]) or \
                abs(float(cdf[want] - target)) < 1e-4 * float(cdf[-1]), (r, got[r], want)
    # all greedy, no scratch
    ops().sample(logits, None, None, None, None, out, None)
    assert out.tolist() == logits.argmax(-1).tolist()


# ------------------------------------------------------ decode attention (mma)
DECODE_CASES = [
    # nq, nkv, d, P, single-token segments at positions, window, standout (segment, key)
    (6, 1, 128, 64, [0, 1, 63, 64, 200], None, None),
    (48, 8, 128, 64, [2047, 100], None, (0, 5)),          # far key among thousands
    (4, 2, 32, 4, [37, 9], 6, None),                      # window edge inside small pages
    (12, 2, 64, 16, [700], None, (0, 333)),               # one row: many splits
    (40, 2, 64, 32, [130, 64], 100, None),                # group of 20: two head tiles
    (3, 3, 32, 8, [300, 5, 77], None, None),              # group of 1
    # pages of a multiple of 64 and head size 64 / 128: tiles fetched by TMA
    (8, 2, 64, 128, [500, 64, 127, 128], None, (0, 70)),   # two tiles in a page
    (12, 4, 128, 64, [900, 3], 150, None),                # window over three pages
    (40, 2, 64, 64, [130, 64], 100, None),                # group of 20: two head tiles
]


@pytest.mark.parametrize("nq,nkv,d,P,positions,window,standout", DECODE_CASES)
def test_attn_decode(nq, nkv, d, P, positions, window, standout):
    from freetoken_b200.parts.base import Workspace
    o = ops()
    lens = [(p, 1) for p in positions]
    q, kv, pos, seg, table = _paged_case("bfloat16", nq, nkv, d, P, lens, window, standout=standout)
    out = torch.zeros_like(q)
    scale = d ** -0.5
    o.attn_decode(q, out, kv, None, len(positions), pos, seg, table, nq, nkv, d, scale, window,
                  max(positions) + 1, Workspace(DEV))
    want = _attn_ref(q, kv, pos, seg, table, nq, nkv, d, P, scale, window)
    assert torch.allclose(out.float().cpu(), want, **TOL["bfloat16"])
    o.check_tc_status(DEV)
    if d in (64, 128) and P % 64 == 0:
        # the same through the cp.async kernel, and through the TMA-fed kernel with the
        # splits merged by the separate kernel instead of by a cluster
        for name in ("DECODE_TMA", "DECODE_CLUSTER"):
            out3 = torch.zeros_like(q)
            setattr(o, name, False)
            try:
                o.attn_decode(q, out3, kv, None, len(positions), pos, seg, table, nq, nkv, d, scale, window,
                              max(positions) + 1, Workspace(DEV))
            finally:
                setattr(o, name, True)
            assert torch.allclose(out3.float().cpu(), want, **TOL["bfloat16"]), name
    # a subset of rows through the row list leaves the other rows alone
    if len(positions) > 1:
        rows = torch.tensor([len(positions) - 1], dtype=torch.int32, device=DEV)
        out2 = torch.full_like(q, 7.0)
        o.attn_decode(q, out2, kv, rows, 1, pos, seg, table, nq, nkv, d, scale, window,
                      positions[-1] + 1, Workspace(DEV))
        assert torch.allclose(out2[-1].float().cpu(), want[-1], **TOL["bfloat16"])
        assert (out2[:-1] == 7.0).all()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("T,E,H", [(1, 4, 64), (8, 256, 3072), (33, 37, 104)])
def test_router_logits(dtype, T, E, H):
    x = rnd(T, H, dtype=DT[dtype], seed=1)
    w = rnd(E, H, seed=2, scale=0.05)
    out = torch.empty(T, E, device=DEV)
    ops().router_logits(x, w, out)
    assert torch.allclose(out, x.float() @ w.t(), atol=1e-4, rtol=1e-5)


# ----------------------------------------------------- prefill attention (mma)
PREFILL_CASES = [
    # nq, nkv, d, P, segments (pos0, n), window, standout
    (6, 1, 128, 64, [(0, 70)], None, None),
    (4, 2, 64, 16, [(0, 3), (17, 2), (100, 130)], None, (2, 7)),   # far key, prefix in the cache
    (12, 2, 32, 4, [(5, 64), (0, 65)], None, None),                 # tile edges: 64 and 65 tokens
    (4, 4, 64, 8, [(30, 90)], 20, None),                            # window shorter than a tile
    (8, 2, 128, 64, [(1000, 2), (0, 2)], None, (0, 500)),           # two-token portions
]


@pytest.mark.parametrize("nq,nkv,d,P,lens,window,standout", PREFILL_CASES)
def test_attn_prefill(nq, nkv, d, P, lens, window, standout):
    o = ops()
    q, kv, pos, seg, table = _paged_case("bfloat16", nq, nkv, d, P, lens, window, standout=standout)
    out = torch.zeros_like(q)
    scale = d ** -0.5
    starts = [0]
    for _, n in lens:
        starts.append(starts[-1] + n)
    tiles = [(s, q0) for s, (_, n) in enumerate(lens) for q0 in range(0, n, 64)]
    dev = lambda xs: torch.tensor(xs, dtype=torch.int32, device=DEV)
    o.attn_prefill(q, out, kv, dev([t[0] for t in tiles]), dev([t[1] for t in tiles]), dev(starts),
                   dev([p for p, _ in lens]), table, nq, nkv, d, scale, window)
    want = _attn_ref(q, kv, pos, seg, table, nq, nkv, d, P, scale, window)
    assert torch.allclose(out.float().cpu(), want, **TOL["bfloat16"])


# ------------------------------------------- prefill attention (tcgen05 + TMA)
PREFILL_TC_CASES = [
    # nq, nkv, d, P, segments (pos0, n), standout
    (6, 1, 128, 64, [(0, 70)], None),
    (4, 2, 128, 64, [(0, 3), (200, 130), (64, 257)], (1, 7)),      # far key, prefix in the cache
    (5, 5, 64, 64, [(5, 128), (0, 129)], None),                     # tile edges: 128 and 129 tokens
    (8, 2, 64, 128, [(100, 300)], (0, 2)),                          # two key tiles in a page
    (4, 2, 128, 64, [(1000, 2), (0, 2), (0, 330)], (0, 500)),       # two-token portions beside a long one
]


@pytest.mark.parametrize("nq,nkv,d,P,lens,standout", PREFILL_TC_CASES)
def test_attn_prefill_tc(nq, nkv, d, P, lens, standout):
    o = ops()
    q, kv, pos, seg, table = _paged_case("bfloat16", nq, nkv, d, P, lens, None, standout=standout)
    out = torch.zeros_like(q)
    scale = d ** -0.5
    starts = [0]
    for _, n in lens:
        starts.append(starts[-1] + n)
    tiles = [(s, q0) for s, (_, n) in enumerate(lens) for q0 in range(0, n, 64)]
    dev = lambda xs: torch.tensor(xs, dtype=torch.int32, device=DEV)
    assert o.attn_prefill_tc_takes(q, kv, d, None)
    o.attn_prefill_tc(q, out, kv, dev([t[0] for t in tiles]), dev([t[1] for t in tiles]), dev(starts),
                      dev([p for p, _ in lens]), table, nq, nkv, d, scale)
    o.check_tc_status(DEV)
    want = _attn_ref(q, kv, pos, seg, table, nq, nkv, d, P, scale, None)
    assert torch.allclose(out.float().cpu(), want, **TOL["bfloat16"])


def test_patch_tokens_copies_sampled_ids_into_the_next_steps_inputs():
    o = ops()
    ids = torch.arange(100, 120, dtype=torch.int32, device=DEV)
    src = torch.tensor([7, 8, 999999, -3, 11], dtype=torch.int32, device=DEV)
    rows = torch.tensor([0, 19, 5, 6, 7], dtype=torch.int32, device=DEV)
    src_index = torch.tensor([4, 0, 2, 3, 1], dtype=torch.int32, device=DEV)
    o.patch_tokens(ids, rows, src, src_index, 1000)
    want = list(range(100, 120))
    want[0], want[19], want[5], want[6], want[7] = 11, 7, 0, 0, 8     # ids outside the vocabulary become 0
    assert ids.tolist() == want
