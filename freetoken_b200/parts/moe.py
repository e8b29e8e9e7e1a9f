"""Top-k routed gated-linear-unit experts.

Router, all float32 (python/freetoken/models/minimax_m3/moe.py:71-81;
softmax variant python/freetoken/moe/fused.py:27-31):
``logits = x @ Wg^T``; ``s = sigmoid(logits)`` or ``softmax(logits)``;
experts are chosen by ``s + bias`` (the bias only chooses), weights are the
unbiased ``s`` of the chosen, optionally renormalised to sum 1, times ``scale``.

Experts (python/freetoken/moe/fused.py:267-337,
python/freetoken/layers/moe.py:83-92): routes are sorted by expert;
``m = act(Wgate_e x) * (Wup_e x)`` from one product against ``[gate; up]``;
``y_route = w_route * (Wdown_e m)`` with the weight applied to the float32
accumulator; ``y = sum over the k routes`` in float32, slot order.
Activation ``silu`` or ``swigluoai``
(python/freetoken/kernel/triton/activation.py:96-107).
"""

from __future__ import annotations

from typing import Dict, List

import torch

from ..csrc import ops
from ..weights.spec import Cat, Init, Name, Stack, TensorSpec
from . import linear
from .base import FeedForward, StepContext, register_feed_forward


# Above this many rows per expert (on average) the experts run on the tcgen05
# grouped GEMM; below it the weight-streaming kernel reads each expert once.
# Measured on a B200 with 256 experts, top-8 (decode batches of 32 .. 512): at an
# average of 4 rows the two are level, at 6 the grouped GEMM is 6 % ahead, at 8 rows
# 20 % (the streaming kernel then reads many experts twice, 8 rows a pass).
TC_MIN_ROWS_PER_EXPERT = 4

# Up to this many tokens the router's logits come from the one-warp-per-expert
# kernel; above it from the tiled float32 product.
ROUTER_SMALL_T = 64


def bf16_terms(w: torch.Tensor) -> torch.Tensor:
    """``[terms * E, H]`` bfloat16 whose ``terms`` row blocks sum exactly to the
    float32 matrix ``w``: hi = bf16(w), mid = bf16(w - hi), lo = bf16(w - hi - mid)
    (three 8-bit pieces cover a 24-bit significand; the differences are exact in
    float32).  A product of bfloat16 activations with each term is exact in
    float32, so a tensor-core product with float32 accumulation over the terms
    computes the float32 router logits without rounding the weight."""
    if w.dtype == torch.bfloat16:
        return w
    terms, rest = [], w.float()
    for _ in range(3):
        t = rest.to(torch.bfloat16)
        terms.append(t)
        rest = rest - t.float()
    return torch.cat(terms, 0).contiguous()


@register_feed_forward("routed_experts")
class RoutedExperts(FeedForward):
    """params: ``hidden_size, intermediate_size, num_experts, top_k, scoring``
    (sigmoid | softmax), ``use_bias, renormalize, scale, activation`` (silu |
    swigluoai), ``act_alpha, act_limit, scope`` and ``checkpoint_names``
    (router, bias, gate_up, down: model-side names below the scope; gate, up,
    down_each: per-expert checkpoint names with ``{e}``)."""

    graph_capturable = True

    def __init__(self, spec, prefix):
        super().__init__(spec, prefix)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.inter = int(p["intermediate_size"])
        self.E = int(p["num_experts"])
        self.k = int(p["top_k"])
        self.softmax = p.get("scoring", "sigmoid") == "softmax"
        self.use_bias = bool(p.get("use_bias", False))
        self.renorm = bool(p.get("renormalize", True))
        self.scale = float(p.get("scale", 1.0))
        self.act = p.get("activation", "silu")
        self.act_alpha = float(p.get("act_alpha", 1.702))
        self.act_limit = float(p.get("act_limit", 7.0))
        if self.k > self.E:
            raise ValueError(f"top_k {self.k} exceeds num_experts {self.E}")
        names = p["checkpoint_names"]
        self.scope = self.name(p["scope"])
        self.n_router = f"{self.scope}.{names['router']}"
        self.n_bias = f"{self.scope}.{names['bias']}"
        self.n_gate_up = f"{self.scope}.{names['gate_up']}"
        self.n_down = f"{self.scope}.{names['down']}"
        self._each = {key: f"{self.scope}.{names[key]}" for key in ("gate", "up", "down_each")}
        self.w_router = self.w_router_terms = self.w_bias = self.w_gate_up = self.w_down = None

    def tensor_specs(self) -> List[TensorSpec]:
        E, I, H = self.E, self.inter, self.hidden
        gate_up = Stack(tuple(
            Cat((Name(self._each["gate"].format(e=e), (I, H)),
                 Name(self._each["up"].format(e=e), (I, H))), 0) for e in range(E)))
        down = Stack(tuple(Name(self._each["down_each"].format(e=e), (H, I)) for e in range(E)))
        return [
            TensorSpec(self.n_router, (E, H), role="small32", keep_float32_in_file=True),
            TensorSpec(self.n_bias, (E,), role="small32", keep_float32_in_file=True,
                       init=Init(0.0, 0.01 if self.use_bias else 0.0), tag="router_bias",
                       optional=not self.use_bias),
            TensorSpec(self.n_gate_up, (E, 2 * I, H), sources=(gate_up,)),
            TensorSpec(self.n_down, (E, H, I), sources=(down,), tag="residual_out"),
        ]

    def bind(self, tensors: Dict[str, torch.Tensor], dtype) -> None:
        self.w_router = tensors[self.n_router]
        self.w_router_terms = bf16_terms(self.w_router) if dtype == torch.bfloat16 else None
        # The bias is part of the routing whenever the checkpoint carries it: the
        # reference's block always adds it (python/freetoken/models/minimax_m3/moe.py:75,
        # weight.py:220).  ``use_bias`` only decides whether its absence is an error.
        self.w_bias = tensors.get(self.n_bias)
        self.w_gate_up = tensors[self.n_gate_up]
        self.w_down = tensors[self.n_down]

    def libraries(self, dtype) -> List[str]:
        libs = ["gemm_simt", "moe_route", "elementwise"]
        return libs + (["skinny_gemm", "moe_gemm_tc"] if dtype == torch.bfloat16 else [])

    # ---- forward ----------------------------------------------------------------
    def route(self, ctx: StepContext, x: torch.Tensor, sort_into=None):
        """``(ids [T,k] int32, weights [T,k] float32)``.  With ``sort_into``
        (counts, offsets, sorted_route, sorted_token, active) the routes may be
        sorted as well: returns ``(ids, weights, sorted?)``, the flag saying
        whether that was done here (a handful of tokens: one launch for both)."""
        T = x.shape[0]
        ws = ctx.workspace
        logits = ws.get("moe.logits", (T, self.E), torch.float32)
        terms = 1
        if ctx.dtype == torch.bfloat16 and T <= ROUTER_SMALL_T and ops.router_logits_takes(x, self.w_router):
            ops.router_logits(x, self.w_router, logits)
        elif ctx.dtype == torch.bfloat16 and self.w_router_terms is not None and linear.library_f32_out(
                x, self.w_router_terms, ws.get("moe.logit_terms", (T, self.w_router_terms.shape[0]),
                                               torch.float32)):
            # many rows: tensor-core products of the bfloat16 activations with the exact
            # bfloat16 terms of the float32 router weight; the terms are summed by the selection
            terms = self.w_router_terms.shape[0] // self.E
            logits = ws.get("moe.logit_terms", (T, self.w_router_terms.shape[0]), torch.float32)
        else:
            ops.gemm_rows(x, self.w_router, logits)
        ids = ws.get("moe.ids", (T, self.k), torch.int32)
        weights = ws.get("moe.weights", (T, self.k), torch.float32)
        if sort_into is not None and ops.route_small_takes(T, self.E, self.k):
            ops.route_small(logits, self.w_bias, ids, weights, *sort_into, self.k, self.softmax,
                            self.renorm, self.scale, terms)
            return ids, weights, True
        ops.router_select(logits, self.w_bias, ids, weights, self.k, self.softmax, self.renorm,
                          self.scale, terms)
        return (ids, weights) if sort_into is None else (ids, weights, False)

    def forward(self, ctx: StepContext, x: torch.Tensor) -> torch.Tensor:
        T = x.shape[0]
        R = T * self.k
        ws = ctx.workspace
        counts = ws.get("moe.counts", (self.E,), torch.int32)
        offsets = ws.get("moe.offsets", (self.E + 1,), torch.int32)
        sorted_route = ws.get("moe.sorted_route", (R,), torch.int32)
        sorted_token = ws.get("moe.sorted_token", (R,), torch.int32)
        active = ws.get("moe.active", (self.E + 1,), torch.int32)
        ids, weights, is_sorted = self.route(ctx, x, (counts, offsets, sorted_route, sorted_token, active))
        if not is_sorted:
            scratch = None
            if R >= ops.MOE_SORT_CHUNKED_FROM:
                scratch = ws.get("moe.sort_scratch", (ops.moe_sort_scratch(R, self.E),), torch.int32)
            ops.moe_sort(ids.view(-1), counts, offsets, sorted_route, sorted_token, active, self.E,
                         self.k, scratch)
        if ctx.probe is not None:
            if "router_ids" in ctx.probe:
                ctx.probe["router_ids"].append(ids.clone())
            else:
                ctx.probe.setdefault("experts_touched", []).append(int((counts > 0).sum()))
        mid = ws.get("moe.mid", (R, self.inter), ctx.dtype)
        parts = ws.get("moe.parts", (R, self.hidden), ctx.dtype)
        self.experts(ctx, x, mid, parts, offsets, active, sorted_route, sorted_token,
                     weights.view(-1), R)
        # the k partial rows of a token are summed by whoever consumes them
        # (the next norm adds them into the residual in slot order)
        return parts.view(T, self.k, self.hidden)

    def experts(self, ctx, x, mid, parts, offsets, active, sorted_route, sorted_token, route_weight, R):
        if ctx.dtype == torch.bfloat16 and R > TC_MIN_ROWS_PER_EXPERT * self.E \
                and ops.moe_gemm_tc_takes(x, self.w_gate_up, mid) \
                and ops.moe_gemm_tc_takes(mid, self.w_down, parts):
            # many rows per expert: tcgen05 grouped GEMM over the rows sorted by expert
            ops.moe_experts_tc(x, self.w_gate_up, self.w_down, mid, parts, offsets, active, sorted_route,
                               sorted_token, route_weight, R, self.act, self.act_alpha, self.act_limit,
                               ctx.workspace)
            return
        if ctx.dtype == torch.bfloat16 and ops.skinny_gemm_takes(x, self.w_gate_up, mid) \
                and ops.skinny_gemm_takes(mid, self.w_down, parts):
            per_pass = ops.pass_rows(-(-R // self.E))
            ops.skinny_gemm(x, self.w_gate_up, mid, group_offsets=offsets, active=active,
                            a_rows=sorted_token,
                            rows=R, glu=True, act=self.act, act_alpha=self.act_alpha,
                            act_limit=self.act_limit, rows_per_pass=per_pass)
            ops.skinny_gemm(mid, self.w_down, parts, group_offsets=offsets, active=active,
                            c_rows=sorted_route,
                            row_scale=route_weight, rows=R, rows_per_pass=per_pass)
            return
        ops.gemm_rows(x, self.w_gate_up, mid, group_offsets=offsets, a_rows=sorted_token, rows=R,
                      glu=True, act=self.act, act_alpha=self.act_alpha, act_limit=self.act_limit)
        ops.gemm_rows(mid, self.w_down, parts, group_offsets=offsets, c_rows=sorted_route,
                      row_scale=route_weight, rows=R)
