"""A plain, slow implementation of the MiniMax-M3 decoder, for comparison only.

Whole sequences, no cache, no batching, one function per part, PyTorch on the
CPU.  It shares no code with ``freetoken_b200``: it reads ``config.json`` and
``model.safetensors`` itself and is written from the reference's formulas, each
cited as ``file:line`` below (paths inside TaoLe-si/FreeToken).

The reference's model code cannot run here as a whole: ``import
freetoken.models`` needs the absent ``flashlib`` package, its rotary module
refuses head sizes other than 64/128/256/512 (python/freetoken/layers/rotary.py:60),
and its ``minimax_m3`` module hard-wires options this decoder reads from
config.json.  Its pieces do run, and every part below is compared with them
once (``tests/golden/``, ``tests/test_plain_model.py``): the router's ``_route``
and the rotary table on the CPU, and - run once on a GPU - the reference's own
Triton kernels for the rotation (both pairings), the add + RMSNorm (plain and
1+w, per-head), the gated activations, paged causal attention and the whole
``fused_experts_impl``.

Precision: ``compute="float32"`` does everything in float32 on the stored
values.  ``compute="bfloat16"`` rounds activations to bfloat16 wherever a
bfloat16 pipeline stores them (projection outputs, norm outputs, attention
output, expert intermediates), while softmax, norms, router, rotation and the
residual stream stay float32.
"""

from __future__ import annotations

import json
import os
import struct
from typing import Dict, List, Optional, Tuple

import torch


# ----------------------------------------------------------------- reading
_ST_DTYPES = {"F32": torch.float32, "BF16": torch.bfloat16, "F16": torch.float16,
              "I32": torch.int32, "I64": torch.int64}


def read_safetensors(path: str) -> Dict[str, torch.Tensor]:
    """8-byte header length, JSON header, raw little-endian data."""
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        data = f.read()
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        a, b = meta["data_offsets"]
        t = torch.frombuffer(bytearray(data[a:b]), dtype=_ST_DTYPES[meta["dtype"]])
        out[name] = t.reshape(meta["shape"]).clone()
    return out


def read_model(folder: str) -> Tuple[dict, Dict[str, torch.Tensor]]:
    with open(os.path.join(folder, "config.json")) as f:
        config = json.load(f)
    return config, read_safetensors(os.path.join(folder, "model.safetensors"))


# ------------------------------------------------------------------- parts
def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float, plus_one: bool) -> torch.Tensor:
    """y = x * rsqrt(mean(x^2) + eps) * w, float32; (1 + w) for the Gemma form.
    python/freetoken/kernel/triton/norm.py:65-75 (plain), :69-72 (1+w)."""
    x = x.float()
    w = w.float() + (1.0 if plus_one else 0.0)
    inv = torch.rsqrt(x.pow(2).mean(dim=-1, keepdim=True) + eps)
    return x * inv * w


def rope_table(num_positions: int, rotary_dim: int, theta: float) -> Tuple[torch.Tensor, torch.Tensor]:
    """inv_freq_i = theta^(-2i/R); cos/sin of position * inv_freq, float32.
    python/freetoken/layers/rotary.py:49-59."""
    inv_freq = 1.0 / (theta ** (torch.arange(0, rotary_dim, 2, dtype=torch.float) / rotary_dim))
    t = torch.arange(num_positions, dtype=torch.float)
    freqs = torch.einsum("i,j -> ij", t, inv_freq)
    return freqs.cos(), freqs.sin()


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, rotary_dim: int) -> torch.Tensor:
    """NeoX pairing on the first rotary_dim dims of every head; the rest passes.
    x: [T, heads, d]; cos, sin: [T, rotary_dim/2].
    x_i' = x_i cos_i - x_{i+R/2} sin_i ; x_{i+R/2}' = x_{i+R/2} cos_i + x_i sin_i
    python/freetoken/kernel/triton/rope.py:62-64,73-78."""
    if rotary_dim == 0:
        return x
    half = rotary_dim // 2
    x = x.float().clone()
    x0 = x[..., :half].clone()
    x1 = x[..., half:rotary_dim].clone()
    c = cos[:, None, :]
    s = sin[:, None, :]
    x[..., :half] = x0 * c - x1 * s
    x[..., half:rotary_dim] = x1 * c + x0 * s
    return x


def qk_norm(q: torch.Tensor, k: torch.Tensor, qw, kw, mode: str, eps: float, plus_one: bool,
            nq: int, nkv: int, d: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """per_layer: one RMSNorm over the whole q (nq*d) and whole k (nkv*d) row,
    python/freetoken/models/minimax_m2/attention.py:45-47,78-79.
    per_head: one RMSNorm per head over d with a [d] weight shared by all heads,
    python/freetoken/models/minimax_m3/attention.py:54-56,90-91.  v is never normed."""
    if mode == "none":
        return q.float(), k.float()
    if mode == "per_layer":
        return rms_norm(q, qw, eps, plus_one), rms_norm(k, kw, eps, plus_one)
    T = q.shape[0]
    qh = rms_norm(q.view(T, nq, d), qw, eps, plus_one).reshape(T, nq * d)
    kh = rms_norm(k.view(T, nkv, d), kw, eps, plus_one).reshape(T, nkv * d)
    return qh, kh


def causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
                     window: Optional[int] = None) -> torch.Tensor:
    """s_tj = (q_t . k_j) * scale for j <= t (and j > t - window), softmax over j,
    o_t = sum_j p_tj v_j; query head h reads KV head h // group.
    python/freetoken/kernel/triton/attention.py:74,118-139,191; scale = d^-0.5
    python/freetoken/attention/triton.py:163.   q: [T,nq,d]; k,v: [T,nkv,d]."""
    T, nq, d = q.shape
    nkv = k.shape[1]
    group = nq // nkv
    out = torch.zeros(T, nq, d, dtype=torch.float32)
    pos = torch.arange(T)
    mask = pos[None, :] <= pos[:, None]
    if window is not None:
        mask &= pos[None, :] > pos[:, None] - window
    for h in range(nq):
        kh, vh = k[:, h // group].float(), v[:, h // group].float()
        s = (q[:, h].float() @ kh.t()) * scale
        s = s.masked_fill(~mask, float("-inf"))
        p = torch.softmax(s, dim=-1)
        out[:, h] = p @ vh
    return out


def route(h: torch.Tensor, gate_w: torch.Tensor, bias: Optional[torch.Tensor], top_k: int,
          scoring: str, renormalize: bool, scale: float, forced_ids: Optional[torch.Tensor] = None,
          record: Optional[list] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """logits = h.float() @ Wg.float()^T; s = sigmoid(logits); choose top-k of s + bias;
    weights = s[ids] (unbiased); w /= (sum w + 1e-20); w *= scale.
    python/freetoken/models/minimax_m3/moe.py:71-81.
    softmax variant: s = softmax(logits), top-k of s, python/freetoken/moe/fused.py:27-31.
    Ties go to the lower expert id (torch.topk leaves the order open).
    ``forced_ids`` replaces the choice (weights still come from this function's
    own scores); ``record`` receives ``(own ids, margin of the own choice)``."""
    logits = h.float() @ gate_w.float().t()
    s = torch.softmax(logits, dim=-1) if scoring == "softmax" else torch.sigmoid(logits)
    choice = s + (bias.float() if bias is not None else 0.0)
    T, E = choice.shape
    ids = torch.empty(T, top_k, dtype=torch.long)
    c = choice.clone()
    for j in range(top_k):
        best = c.max(dim=-1, keepdim=True).values
        first = (c == best).float().argmax(dim=-1)   # lowest index among equals
        ids[:, j] = first
        c[torch.arange(T), first] = float("-inf")
    if record is not None:
        # own choice and its margin: k-th chosen value minus the best value left out
        kth = choice.gather(-1, ids[:, -1:]).squeeze(-1)
        left = c.max(dim=-1).values if top_k < E else torch.full((T,), float("-inf"))
        record.append((ids.clone(), kth - left))
    if forced_ids is not None:
        ids = forced_ids.long()
    w = s.gather(-1, ids)
    if renormalize:
        w = w / (w.sum(dim=-1, keepdim=True) + 1e-20)
    return w * scale, ids


def glu(g: torch.Tensor, u: torch.Tensor, act: str, alpha: float, limit: float) -> torch.Tensor:
    """silu(g) * u, python/freetoken/kernel/triton/activation.py:96-98;
    swigluoai: min(g,L) * sigmoid(alpha * min(g,L)) * (clamp(u,-L,L) + 1), :103-107."""
    if act == "silu":
        return torch.nn.functional.silu(g) * u
    g = g.clamp(max=limit)
    u = u.clamp(min=-limit, max=limit)
    return g * torch.sigmoid(alpha * g) * (u + 1.0)


def experts(h: torch.Tensor, w: torch.Tensor, ids: torch.Tensor, gate_up: List[torch.Tensor],
            down: List[torch.Tensor], act: str, alpha: float, limit: float,
            round_to, round_gate_up=None) -> torch.Tensor:
    """y_t = sum_j w_tj * Wdown_e ( act(Wgate_e h_t) * (Wup_e h_t) ), e = ids_tj.
    [gate; up] halves un-interleaved, python/freetoken/layers/activation.py:50-53;
    the route weight multiplies the float32 product before rounding,
    python/freetoken/kernel/triton/fused_moe.py:292-296; the k terms are summed in
    float32, fused_moe.py:143-153.  ``round_gate_up`` (when given) rounds the
    [gate; up] product before the activation, as the reference does by storing it
    in the activation dtype (python/freetoken/moe/fused.py:268-300); the engine's
    kernels feed the activation from the float32 accumulator instead."""
    T, H = h.shape
    out = torch.zeros(T, H, dtype=torch.float32)
    for t in range(T):
        acc = torch.zeros(H, dtype=torch.float32)
        for j in range(ids.shape[1]):
            e = int(ids[t, j])
            gu = gate_up[e].float() @ h[t].float()
            if round_gate_up is not None:
                gu = round_gate_up(gu)
            inter = gu.shape[0] // 2
            m = round_to(glu(gu[:inter], gu[inter:], act, alpha, limit))
            y = round_to((down[e].float() @ m.float()) * w[t, j])
            acc = acc + y.float()
        out[t] = acc
    return out


# ------------------------------------------------------------------- model
class PlainModel:
    def __init__(self, folder: str, compute: str = "float32"):
        self.config, self.tensors = read_model(folder)
        self.compute = compute
        c = self.config.get("text_config") or self.config
        self.c = c
        self.H = c["hidden_size"]
        self.L = c["num_hidden_layers"]
        self.nq = c["num_attention_heads"]
        self.nkv = c.get("num_key_value_heads", self.nq)
        self.d = c.get("head_dim") or self.H // self.nq      # args.py:212-214
        self.R = c.get("rotary_dim")
        if self.R is None:                                     # args.py:215-217
            self.R = int(self.d * c.get("partial_rotary_factor", 1.0))
        self.theta = float(c.get("rope_theta", 10000.0))       # args.py:91-96
        self.eps = c["rms_norm_eps"]
        self.plus_one = bool(c.get("use_gemma_norm", True))    # args.py:208-210
        self.qk_mode = c.get("qk_norm_type", "per_head") if c.get("use_qk_norm", True) else "none"
        self.E = c["num_local_experts"]
        self.k = c["num_experts_per_tok"]
        self.scoring = c.get("scoring_func", "sigmoid")
        self.use_bias = bool(c.get("use_routing_bias", False))
        self.renorm = bool(c.get("norm_topk_prob", True))
        self.route_scale = float(c.get("routed_scaling_factor", 1.0))
        self.act = c.get("hidden_act", "swigluoai")
        self.alpha = float(c.get("swiglu_alpha", 1.702))
        self.limit = float(c.get("swiglu_limit", 7.0))
        self.tied = bool(c.get("tie_word_embeddings", False))
        self.window = c.get("sliding_window")
        self.routing: list = []

    def rnd(self, x: torch.Tensor) -> torch.Tensor:
        """Round to the activation dtype of the emulated pipeline."""
        if self.compute == "bfloat16":
            return x.to(torch.bfloat16).float()
        return x.float()

    def w(self, name: str) -> torch.Tensor:
        t = self.tensors[name]
        if self.compute == "bfloat16" and t.dtype == torch.float32 and t.dim() >= 2 \
                and not name.endswith("gate.weight"):
            t = t.to(torch.bfloat16)   # matrices are served in bfloat16; the router's stay float32
        return t.float()

    def layer(self, i: int, x: torch.Tensor, residual: torch.Tensor,
              forced_ids: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
        """(x, residual) in -> (x, residual) out; norms do the adds.
        python/freetoken/models/minimax_m2/model.py:27-37."""
        p = f"model.layers.{i}"
        T = x.shape[0]
        residual = residual + x                                   # norm.py:101-109
        h1 = self.rnd(rms_norm(residual, self.w(f"{p}.input_layernorm.weight"), self.eps, self.plus_one))
        # merged projection, no bias: minimax_m2/attention.py:37-43,76-77
        q = self.rnd(h1 @ self.w(f"{p}.self_attn.q_proj.weight").t())
        k = self.rnd(h1 @ self.w(f"{p}.self_attn.k_proj.weight").t())
        v = self.rnd(h1 @ self.w(f"{p}.self_attn.v_proj.weight").t())
        qw = kw = None
        if self.qk_mode != "none":
            qw = self.w(f"{p}.self_attn.q_norm.weight")
            kw = self.w(f"{p}.self_attn.k_norm.weight")
        q, k = qk_norm(q, k, qw, kw, self.qk_mode, self.eps, self.plus_one, self.nq, self.nkv, self.d)
        cos, sin = rope_table(T, self.R, self.theta) if self.R else (None, None)
        q = self.rnd(apply_rope(q.view(T, self.nq, self.d), cos, sin, self.R))
        k = self.rnd(apply_rope(k.view(T, self.nkv, self.d), cos, sin, self.R))
        o = causal_attention(q, k, v.view(T, self.nkv, self.d), self.d ** -0.5, self.window)
        o = self.rnd(o).reshape(T, self.nq * self.d)
        a = self.rnd(o @ self.w(f"{p}.self_attn.o_proj.weight").t())  # attention.py:84
        residual = residual + a
        h2 = self.rnd(rms_norm(residual, self.w(f"{p}.post_attention_layernorm.weight"), self.eps, self.plus_one))
        m = f"{p}.block_sparse_moe"
        # the block adds the bias whenever the checkpoint has it: minimax_m3/moe.py:75, weight.py:220
        bias = self.tensors[f"{m}.e_score_correction_bias"] if self.use_bias \
            else self.tensors.get(f"{m}.e_score_correction_bias")
        wts, ids = route(h2, self.tensors[f"{m}.gate.weight"], bias, self.k, self.scoring,
                         self.renorm, self.route_scale, forced_ids, self.routing)
        gate_up = [torch.cat([self.w(f"{m}.experts.{e}.w1.weight"), self.w(f"{m}.experts.{e}.w3.weight")])
                   for e in range(self.E)]                        # w1 = gate, w3 = up: weight.py:54
        down = [self.w(f"{m}.experts.{e}.w2.weight") for e in range(self.E)]
        y = self.rnd(experts(h2, wts, ids, gate_up, down, self.act, self.alpha, self.limit, self.rnd))
        return y, residual

    def forward(self, tokens: List[int], forced_routing: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Logits [T, vocab] float32 for the whole sequence.
        python/freetoken/models/minimax_m2/model.py:48-52,66-68.
        ``forced_routing`` ``[layers, T, k]`` fixes the experts every token
        uses; ``self.routing`` afterwards holds, per layer, this model's own
        choice and its margin."""
        self.routing = []
        ids = torch.tensor(tokens, dtype=torch.long)
        emb = self.w("model.embed_tokens.weight")
        residual = emb[ids]                                        # no scale: embedding.py:39-47
        x = torch.zeros_like(residual)
        for i in range(self.L):
            x, residual = self.layer(i, x, residual,
                                     None if forced_routing is None else forced_routing[i])
        xf = self.rnd(rms_norm(residual + x, self.w("model.norm.weight"), self.eps, self.plus_one))
        head = emb if self.tied else self.w("lm_head.weight")      # embedding.py:112
        return xf @ head.t()

    def greedy(self, prompt: List[int], n: int) -> List[int]:
        """Greedy continuation by whole-sequence recomputation (no cache)."""
        seq = list(prompt)
        out = []
        for _ in range(n):
            nxt = int(torch.argmax(self.forward(seq)[-1]))          # engine/sample.py:78-79
            out.append(nxt)
            seq.append(nxt)
        return out
