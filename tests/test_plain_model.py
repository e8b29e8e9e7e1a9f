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
