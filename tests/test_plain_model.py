"""The plain implementation itself: each part against a property or a hand
calculation, and against the two pieces of the reference that run on a CPU."""

import json
import os

import pytest
import torch

import plain_model as pm
import tiny

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "router_rope.json")


def test_router_matches_the_reference_route_function():
    g = json.load(open(GOLDEN))["router"]
    w, ids = pm.route(torch.tensor(g["x"]), torch.tensor(g["gate"]), torch.tensor(g["bias"]),
                      g["top_k"], "sigmoid", True, g["scale"])
    assert ids.tolist() == g["ids"]
    assert torch.allclose(w, torch.tensor(g["weights"]), atol=1e-6, rtol=1e-6)


def test_rope_table_matches_the_reference_table():
    g = json.load(open(GOLDEN))["rope"]
    cos, sin = pm.rope_table(g["positions"], g["rotary_dim"], g["theta"])
    assert torch.equal(torch.cat([cos, sin], -1), torch.tensor(g["cos_sin"]))


def test_rms_norm_forms():
    x = torch.tensor([[3.0, 4.0]])
    w = torch.tensor([0.5, 2.0])
    rms = (12.5 + 1e-6) ** 0.5
    assert torch.allclose(pm.rms_norm(x, w, 1e-6, False), torch.tensor([[1.5 / rms, 8.0 / rms]]))
    assert torch.allclose(pm.rms_norm(x, w, 1e-6, True), torch.tensor([[4.5 / rms, 12.0 / rms]]))


def test_rope_rotates_only_the_leading_dims_and_keeps_norms():
    T, h, d, R = 5, 2, 12, 8
    x = torch.randn(T, h, d)
    cos, sin = pm.rope_table(T, R, 1e4)
    y = pm.apply_rope(x, cos, sin, R)
    assert torch.equal(y[..., R:], x[..., R:])
    assert torch.allclose(y[0], x[0])                                  # position 0: no rotation
    assert torch.allclose(y[..., :R].norm(dim=-1), x[..., :R].norm(dim=-1), atol=1e-5)
    # relative position: <rope(q,m), rope(k,n)> depends on m - n only
    q, k = torch.randn(1, 1, R), torch.randn(1, 1, R)
    c9, s9 = pm.rope_table(10, R, 1e4)
    def at(v, p): return pm.apply_rope(v, c9[p:p + 1], s9[p:p + 1], R)
    assert torch.allclose((at(q, 7) * at(k, 4)).sum(), (at(q, 5) * at(k, 2)).sum(), atol=1e-5)


def test_attention_is_causal_grouped_and_windowed():
    T, nq, nkv, d = 7, 4, 2, 8
    q, k, v = torch.randn(T, nq, d), torch.randn(T, nkv, d), torch.randn(T, nkv, d)
    full = pm.causal_attention(q, k, v, d ** -0.5)
    assert torch.allclose(full[0], v[0].repeat_interleave(2, 0))        # first token sees itself only
    k2, v2 = k.clone(), v.clone()
    k2[5:], v2[5:] = 9.0, -3.0
    assert torch.allclose(pm.causal_attention(q, k2, v2, d ** -0.5)[:5], full[:5])   # the future is invisible
    win = pm.causal_attention(q, k, v, d ** -0.5, window=1)
    assert torch.allclose(win, v.repeat_interleave(2, 1))               # window 1: own value
    # heads 0,1 read KV head 0; heads 2,3 read KV head 1
    v3 = v.clone(); v3[:, 1] = 0
    out3 = pm.causal_attention(q, k, v3, d ** -0.5)
    assert torch.allclose(out3[:, :2], full[:, :2]) and (out3[:, 2:] == 0).all()


def test_router_options_and_ties():
    h = torch.zeros(1, 4)
    gate = torch.zeros(6, 4)
    w, ids = pm.route(h, gate, None, 3, "sigmoid", True, 1.0)
    assert ids.tolist() == [[0, 1, 2]]                                   # ties: lower ids
    assert torch.allclose(w, torch.full((1, 3), 1 / 3))
    w, _ = pm.route(h, gate, None, 3, "softmax", False, 1.5)
    assert torch.allclose(w, torch.full((1, 3), 1.5 / 6))                # softmax over all 6, not renormalised
    bias = torch.tensor([0., 0., 0., 0., 1., 0.])
    w, ids = pm.route(h, gate, bias, 2, "sigmoid", False, 1.0)
    assert ids.tolist() == [[4, 0]] and torch.allclose(w, torch.full((1, 2), 0.5))   # bias chooses, not weighs


def test_glu_forms():
    g, u = torch.tensor([1.0, 9.0]), torch.tensor([2.0, -8.0])
    assert torch.allclose(pm.glu(g, u, "silu", 0, 0), torch.nn.functional.silu(g) * u)
    got = pm.glu(g, u, "swigluoai", 1.702, 7.0)
    want = torch.tensor([1.0 * torch.sigmoid(torch.tensor(1.702)) * 3.0,
                         7.0 * torch.sigmoid(torch.tensor(1.702 * 7.0)) * (-7.0 + 1.0)])
    assert torch.allclose(got, want)


@pytest.mark.parametrize("which", ["A", "B"])
def test_whole_model_properties(tmp_path, which):
    folder = tiny.write_tiny(str(tmp_path), which)
    model = pm.PlainModel(folder, "float32")
    vocab = tiny.TINY[which]["vocab_size"]
    toks = tiny.tokens(3, 12, vocab)
    logits = model.forward(toks)
    assert logits.shape == (12, vocab) and torch.isfinite(logits).all()
    forced = torch.stack([r[0] for r in model.routing])
    assert torch.allclose(model.forward(toks[:7]), logits[:7], atol=1e-5)      # causal: prefixes agree
    assert torch.equal(model.forward(toks, forced), model.forward(toks))       # forcing the own choice changes nothing
    bf = pm.PlainModel(folder, "bfloat16").forward(toks)
    assert torch.allclose(bf, logits, atol=3e-2, rtol=3e-2) and not torch.equal(bf, logits)
    out = model.greedy(toks[:4], 3)
    assert len(out) == 3 and all(0 <= t < vocab for t in out)


# ------------------------------------------------------------------------------
# The plain implementation's parts against outputs of the reference's own Triton
# kernels (tests/golden/make_kernel_golden.py ran them once on a GPU; inputs and
# outputs are in tests/golden/triton_kernels.safetensors).
KERNEL_GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "triton_kernels.safetensors")


@pytest.fixture(scope="module")
def kg():
    return pm.read_safetensors(KERNEL_GOLDEN)


def test_kernel_golden_file_covers_all_five_kernels():
    import struct
    with open(KERNEL_GOLDEN, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        meta = json.loads(f.read(n))["__metadata__"]
    for name in ("rope", "norm", "activation", "attention", "experts"):
        assert meta[name] == "ok", (name, meta[name])


@pytest.mark.parametrize("pairing", ["neox", "interleaved"])
def test_rope_matches_the_reference_kernel(kg, pairing):
    """NeoX halves (i, i + R/2) on the first R dims; kernel/triton/rope.py:59-78."""
    T, d, R = 6, 64, 32
    table = kg["rope.table"][kg["rope.positions"].long()]
    cos, sin = table[:, : R // 2], table[:, R // 2:]
    for name, heads in (("q", 3), ("k", 1)):
        x = kg[f"rope.{name}"].view(T, heads, d)
        want = kg[f"rope.{name}_{pairing}"].view(T, heads, d)
        if pairing == "neox":
            got = pm.apply_rope(x, cos, sin, R)
        else:
            # the (2i, 2i+1) pairing, for the framework's second rotary kind
            got = x.clone()
            x0, x1 = x[..., 0:R:2], x[..., 1:R:2]
            got[..., 0:R:2] = x0 * cos[:, None] - x1 * sin[:, None]
            got[..., 1:R:2] = x1 * cos[:, None] + x0 * sin[:, None]
        assert torch.allclose(got, want, atol=1e-5, rtol=1e-5)
        assert torch.equal(got[..., R:], x[..., R:])
    # the two pairings are different functions: the golden values can tell them apart
    assert not torch.allclose(kg["rope.q_neox"], kg["rope.q_interleaved"], atol=1e-3)


def test_add_rms_norm_matches_the_reference_kernels(kg):
    """residual += x; y = residual * rsqrt(mean^2 + eps) * w  (or 1 + w);
    kernel/triton/norm.py:101-112, :69-72."""
    eps = float(kg["norm.eps"])
    z = kg["norm.x"] + kg["norm.residual"]
    for tag, plus_one in (("plain", False), ("gemma", True)):
        assert torch.allclose(kg[f"norm.{tag}_residual"], z, atol=1e-6)
        w = kg["norm.w"] + (0.0 if plus_one else 1.0)
        assert torch.allclose(pm.rms_norm(z, w, eps, plus_one), kg[f"norm.{tag}_out"], atol=1e-5, rtol=1e-5)
    # per-head norm of q / k: [T, heads, d] with one [d] weight
    T, h, d = kg["norm.heads_x"].shape
    x = kg["norm.heads_x"].reshape(T, h * d)
    q, _ = pm.qk_norm(x, x, kg["norm.heads_w"], kg["norm.heads_w"], "per_head", eps, True, h, h, d)
    assert torch.allclose(q.view(T, h, d), kg["norm.heads_gemma_out"], atol=1e-5, rtol=1e-5)
    q, _ = pm.qk_norm(x, x, kg["norm.heads_w"] + 1.0, kg["norm.heads_w"] + 1.0, "per_head", eps, False, h, h, d)
    assert torch.allclose(q.view(T, h, d), kg["norm.heads_plain_out"], atol=1e-5, rtol=1e-5)


def test_gated_activations_match_the_reference_kernels(kg):
    """[gate | up] halves, gate first; kernel/triton/activation.py:96-107."""
    x = kg["act.x"]
    half = x.shape[1] // 2
    g, u = x[:, :half], x[:, half:]
    assert torch.allclose(pm.glu(g, u, "silu", 0.0, 0.0), kg["act.silu"], atol=1e-5, rtol=1e-5)
    assert torch.allclose(pm.glu(g, u, "swigluoai", 1.702, 7.0), kg["act.swigluoai"], atol=1e-5, rtol=1e-5)
    # gate and up swapped is a different function, so the order is pinned
    assert not torch.allclose(pm.glu(u, g, "silu", 0.0, 0.0), kg["act.silu"], atol=1e-2)


def test_causal_attention_matches_the_reference_kernel(kg):
    """Two requests over shuffled cache slots, one with 9 keys already cached;
    kernel/triton/attention.py:45-145."""
    q, kc, vc = kg["attn.q"], kg["attn.k_cache"], kg["attn.v_cache"]
    indptr, indices = kg["attn.indptr"].tolist(), kg["attn.indices"].long()
    q_pos, q_req = kg["attn.q_pos"].tolist(), kg["attn.q_to_req"].tolist()
    d = q.shape[-1]
    row = 0
    for r in range(len(indptr) - 1):
        slots = indices[indptr[r]: indptr[r + 1]]
        k, v = kc[slots], vc[slots]                       # the request's keys in order
        L = k.shape[0]
        rows = [i for i, rr in enumerate(q_req) if rr == r]
        # the plain function takes whole sequences: pad the queries of cached positions
        full_q = torch.zeros(L, q.shape[1], d)
        for i in rows:
            full_q[q_pos[i]] = q[i]
        want = pm.causal_attention(full_q, k, v, d ** -0.5)
        for i in rows:
            assert torch.allclose(want[q_pos[i]], kg["attn.out"][i], atol=2e-5, rtol=1e-4), (r, i)
        row += len(rows)


def test_experts_match_the_reference_fused_experts(kg):
    """The reference's ``fused_experts_impl`` (moe/fused.py:233-337) in bfloat16:
    w1 = [gate; up], activation, w2, route weight on the float32 product, k-way sum."""
    x, w1, w2 = kg["moe.x"], kg["moe.w1"], kg["moe.w2"]
    ids, wts = kg["moe.ids"].long(), kg["moe.weights"]
    E = w1.shape[0]
    rnd = lambda t: t.to(torch.bfloat16).float()
    # the reference's rounding points: the gate_up product, the activation's output and
    # every route's weighted output are stored in bfloat16, the k-way sum is rounded once more
    got = rnd(pm.experts(x.float(), wts, ids, [w1[e] for e in range(E)], [w2[e] for e in range(E)],
                         "silu", 0.0, 0.0, rnd, round_gate_up=rnd))
    want = kg["moe.out"].float()
    assert want.abs().max() > 4.0
    # with the same rounding points the two differ only where a float32 sum in another
    # order crosses a rounding boundary: one unit in the last place of the largest output
    # (2^-5 for values in [4, 8)), fixed before the comparison was first run
    assert torch.allclose(got, want, atol=2.0 ** -5, rtol=2.0 ** -7), (got - want).abs().max()
    assert (got != want).float().mean() < 0.2
    # swapping gate and up, or dropping the route weight, is far outside that tolerance
    swapped = [torch.cat([w[w.shape[0] // 2:], w[: w.shape[0] // 2]]) for w in w1]
    bad = pm.experts(x.float(), wts, ids, swapped, [w2[e] for e in range(E)], "silu", 0.0, 0.0, rnd)
    assert not torch.allclose(bad, want, atol=0.25, rtol=0.1)
    unweighted = pm.experts(x.float(), torch.ones_like(wts), ids, [w1[e] for e in range(E)],
                            [w2[e] for e in range(E)], "silu", 0.0, 0.0, rnd)
    assert not torch.allclose(unweighted, want, atol=0.25, rtol=0.1)
