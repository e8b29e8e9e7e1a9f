"""Grouped-query softmax attention over the paged cache.

Per token: ``qkv = x @ Wqkv^T`` (one merged product, no bias), optional QK
RMSNorm (over the whole q / k projection, or per head), rotary on the first
``rotary_dim`` dims of each head, K and V stored into the request's pages,
causal softmax attention with scale ``sm_scale`` over the cached keys (all of
them, or the latest ``sliding_window``), then ``@ Wo^T``.

Reference: python/freetoken/models/minimax_m2/attention.py:29-84 (merged QKV,
per-layer norm, rotary, backend call, o_proj),
python/freetoken/models/minimax_m3/attention.py:54-56,90-92 (per-head norm),
python/freetoken/attention/triton.py:150-216 (store, then decode / extend
kernels), python/freetoken/kernel/triton/attention.py:74,118-139 (mask, scale,
softmax).
"""

from __future__ import annotations

from typing import Dict, List

import numpy as np
import torch

from ..cache.manager import PagedKVNeed
from ..csrc import ops
from ..weights.spec import Cat, Init, Name, TensorSpec
from . import linear
from .base import POSITIONS, CacheView, Mixer, StepContext, StepPlan, StepShape, register_mixer

# query tokens per tile of the prefill attention kernels' tile list
PREFILL_TILE = 64

_NORM_MODES = {"none": 0, "per_layer": 1, "per_head": 2}


@register_mixer("paged_attention")
class PagedAttention(Mixer):
    """params: ``hidden_size, num_heads, num_kv_heads, head_dim, sm_scale,
    qk_norm`` (none | per_layer | per_head), ``qk_norm_eps, qk_norm_plus_one,
    sliding_window`` (None: all keys), ``position`` (a PartSpec), ``scope`` and
    ``checkpoint_names`` (q, k, v, o, fused qkv, q_norm, k_norm tensor names
    below the scope)."""

    graph_capturable = True

    def __init__(self, spec, prefix):
        super().__init__(spec, prefix)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.nq = int(p["num_heads"])
        self.nkv = int(p["num_kv_heads"])
        self.d = int(p["head_dim"])
        self.scale = float(p["sm_scale"])
        self.norm_mode = _NORM_MODES[p.get("qk_norm", "none")]
        self.norm_eps = float(p.get("qk_norm_eps", 1e-6))
        self.norm_plus_one = bool(p.get("qk_norm_plus_one", False))
        self.window = p.get("sliding_window")
        if self.nq % self.nkv:
            raise ValueError(f"num_heads {self.nq} is not a multiple of num_kv_heads {self.nkv}")
        if self.d > 256:
            raise ValueError(f"head_dim {self.d} exceeds what the attention kernels take (256)")
        pos_spec = p["position"]
        self.position = POSITIONS.get(pos_spec.kind)(pos_spec, prefix)
        scope = p["scope"]
        names = p["checkpoint_names"]
        self.scope = self.name(scope)
        self.n_qkv = f"{self.scope}.{names['qkv']}"
        self.n_o = f"{self.scope}.{names['o']}"
        self.n_qnorm = f"{self.scope}.{names['q_norm']}"
        self.n_knorm = f"{self.scope}.{names['k_norm']}"
        self._split = [f"{self.scope}.{names[k]}" for k in ("q", "k", "v")]
        self.w_qkv = self.w_o = self.w_qnorm = self.w_knorm = None

    def children(self):
        return [self.position]

    # ---- step metadata ---------------------------------------------------------
    def step_plan_key(self):
        # the lists depend on the step's segments only: every attention layer shares them
        return "paged_attention"

    def plan_step(self, shape: StepShape) -> StepPlan:
        """What the attention kernels want to know about a step: which token rows
        are single-token segments (decode kernel; listed only when the step also
        has longer segments, otherwise it is all rows), the 64-token query tiles
        of the longer segments (prefill kernels: segment and first token inside
        it), how many query-key pairs those score, and the longest context of a
        decode row (in whole block-table rows for a decode-only step, so that the
        split count - and with it a captured graph - stays put while contexts grow)."""
        segs = shape.segments
        dec = [s.q_start for s in segs if s.n == 1]
        tiles = [(i, q0) for i, s in enumerate(segs) if s.n > 1 for q0 in range(0, s.n, PREFILL_TILE)]
        arrays = {
            "tile_seg": np.asarray([t[0] for t in tiles], dtype=np.int32),
            "tile_q0": np.asarray([t[1] for t in tiles], dtype=np.int32),
        }
        if dec and tiles:
            arrays["decode_rows"] = np.asarray(dec, dtype=np.int32)
        if shape.max_q_len == 1:
            max_decode_kv = shape.table_width * shape.page_size
        else:
            max_decode_kv = max((s.pos0 + 1 for s in segs if s.n == 1), default=0)
        host = {
            "num_decode_rows": len(dec),
            "num_prefill_tiles": len(tiles),
            "prefill_scores": sum(s.n * (s.pos0 + (s.n + 1) // 2) for s in segs if s.n > 1),
            "max_decode_kv_len": max_decode_kv,
        }
        return StepPlan(arrays=arrays, host=host)

    # ---- cache and weights ------------------------------------------------
    def cache_need(self):
        return PagedKVNeed(self.nkv, self.d, self.window)

    def tensor_specs(self) -> List[TensorSpec]:
        qn, kn = self.nq * self.d, self.nkv * self.d
        specs = [
            TensorSpec(self.n_qkv, (qn + 2 * kn, self.hidden), sources=(Cat((
                Name(self._split[0], (qn, self.hidden)),
                Name(self._split[1], (kn, self.hidden)),
                Name(self._split[2], (kn, self.hidden))), 0),)),
            TensorSpec(self.n_o, (self.hidden, qn), tag="residual_out"),
        ]
        if self.norm_mode:
            sizes = (qn, kn) if self.norm_mode == 1 else (self.d, self.d)
            mean = 0.0 if self.norm_plus_one else 1.0
            for name, size in zip((self.n_qnorm, self.n_knorm), sizes):
                specs.append(TensorSpec(name, (size,), role="small32",
                                        init=Init(mean=mean, std=0.0), tag="norm"))
        return specs

    def bind(self, tensors: Dict[str, torch.Tensor], dtype) -> None:
        self.w_qkv = tensors[self.n_qkv]
        self.w_o = tensors[self.n_o]
        if self.norm_mode:
            self.w_qnorm = tensors[self.n_qnorm]
            self.w_knorm = tensors[self.n_knorm]

    def libraries(self, dtype) -> List[str]:
        fast = ["attention_decode", "attention_prefill"] if dtype == torch.bfloat16 else []
        if fast and self.d in (64, 128):
            # TMA-fed kernels (the prefill one also builds the tensor maps both use)
            fast += ["attention_prefill_tc", "attention_decode_tma"]
        return ["elementwise", "attention_simt"] + fast + linear.libraries(dtype)

    # ---- forward ----------------------------------------------------------------
    def forward(self, ctx: StepContext, x: torch.Tensor, cache: CacheView) -> torch.Tensor:
        T = x.shape[0]
        ws = ctx.workspace
        qn, kn = self.nq * self.d, self.nkv * self.d
        qkv = linear.linear(x, self.w_qkv, ws.get("attn.qkv", (T, qn + 2 * kn), ctx.dtype))
        q = ws.get("attn.q", (T, qn), ctx.dtype)
        table = ctx.block_tables[cache.block_table_index]
        cos_sin = self.position.table(ctx.device, ctx.max_positions)
        ops.qk_rope_store(
            qkv, q, cache.kv_pages if cache.writes else None, self.w_qnorm, self.w_knorm,
            cos_sin, ctx.token_pos, ctx.token_seg, table, self.nq, self.nkv, self.d,
            self.position.rotary_dim, self.norm_mode, self.norm_plus_one,
            self.position.interleaved, self.norm_eps)
        o = ws.get("attn.o", (T, qn), ctx.dtype)
        self.attend(ctx, q, o, cache, table)
        return linear.linear(o, self.w_o, ws.get("attn.y", (T, self.hidden), ctx.dtype))

    def attend(self, ctx: StepContext, q, o, cache: CacheView, table) -> None:
        """Single-token rows go to the split-KV tensor-core kernel, rows of
        longer segments to a prefill kernel; sizes those refuse (and the
        float32 path) go to the generic kernel."""
        if ops.attn_decode_takes(q, self.d):
            plan = ctx.plan(self)
            n_dec, n_tiles = plan.host["num_decode_rows"], plan.host["num_prefill_tiles"]
            if n_dec > 0:
                ops.attn_decode(q, o, cache.kv_pages, plan.tensors.get("decode_rows"), n_dec,
                                ctx.token_pos, ctx.token_seg, table, self.nq, self.nkv, self.d,
                                self.scale, self.window, plan.host["max_decode_kv_len"], ctx.workspace)
            if n_tiles > 0:
                tile_seg, tile_q0 = plan.tensors["tile_seg"], plan.tensors["tile_q0"]
                if (plan.host["prefill_scores"] >= ops.PREFILL_TC_MIN_SCORES
                        and ops.attn_prefill_tc_takes(q, cache.kv_pages, self.d, self.window)):
                    ops.attn_prefill_tc(q, o, cache.kv_pages, tile_seg, tile_q0, ctx.seg_q_start,
                                        ctx.seg_pos0, table, self.nq, self.nkv, self.d, self.scale)
                    return
                ops.attn_prefill(q, o, cache.kv_pages, tile_seg, tile_q0, ctx.seg_q_start, ctx.seg_pos0,
                                 table, self.nq, self.nkv, self.d, self.scale, self.window)
            return
        ops.attn_paged_simt(q, o, cache.kv_pages, ctx.token_pos, ctx.token_seg, table,
                            self.nq, self.nkv, self.d, self.scale, self.window)
