"""The generic decoder: parts built from a plan, run in the plan's order.

``embed -> for stop in schedule: block(stop.layer) -> final norm -> head`` with
the ``(delta, residual)`` pair carried between blocks
(python/freetoken/models/minimax_m2/model.py:48-52,66-68).  The model owns no
sizes and no cache: parts carry their parameters, the engine hands each stop
its :class:`CacheView`.
"""

from __future__ import annotations

from typing import Dict, Hashable, List, Optional, Sequence

import torch

from ..cache.manager import CacheNeed
from ..config.model_plan import ModelPlan, PartSpec
from ..csrc import ops
from ..parts.base import (BLOCKS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, Block, CacheView, Part,
                          StepContext)
from ..weights.spec import TensorSpec


def _prefix(spec: PartSpec, default: str) -> str:
    return spec.params.get("prefix", default)


def _with_nvtx_range(part: Part, name: str) -> None:
    """Wrap ``part.forward`` in an NVTX range called ``name`` (the reference
    annotates its layers and ops the same way, python/freetoken/utils/torch_utils.py:23-37)."""
    inner = part.forward

    def forward(*args, **kwargs):
        torch.cuda.nvtx.range_push(name)
        try:
            return inner(*args, **kwargs)
        finally:
            torch.cuda.nvtx.range_pop()
    part.forward = forward


class Model:
    def __init__(self, plan: ModelPlan, nvtx: bool = False):
        plan.validate()
        self.plan = plan
        self.embedding = EMBEDDINGS.get(plan.embedding.kind)(plan.embedding, _prefix(plan.embedding, ""))
        self.blocks: List[Block] = []
        for layer in plan.layers:
            # the layer's spec lists what it has; the block kind says what it needs
            block_cls = BLOCKS.get(layer.block.kind)
            norm_specs = layer.all_norms()
            block_cls.check_parts(layer.prefix, sorted(norm_specs), layer.feed_forward is not None)
            mixer = MIXERS.get(layer.mixer.kind)(layer.mixer, layer.prefix)
            ffn = None
            if layer.feed_forward is not None:
                ffn = FEED_FORWARDS.get(layer.feed_forward.kind)(layer.feed_forward, layer.prefix)
            norms = {name: NORMS.get(spec.kind)(spec, layer.prefix) for name, spec in norm_specs.items()}
            self.blocks.append(block_cls(layer.block, layer.prefix, mixer, ffn, norms))
        self.final_norm = NORMS.get(plan.final_norm.kind)(plan.final_norm, _prefix(plan.final_norm, ""))
        self.head = HEADS.get(plan.head.kind)(plan.head, _prefix(plan.head, ""))
        if nvtx:
            for i, block in enumerate(self.blocks):
                _with_nvtx_range(block, f"layer_{i}")
                for child in block.children():
                    _with_nvtx_range(child, f"layer_{i}.{type(child).__name__}")
            for part, name in ((self.embedding, "embedding"), (self.final_norm, "final_norm"), (self.head, "head")):
                _with_nvtx_range(part, name)

    # ---- weights ---------------------------------------------------------
    def parts(self):
        return [self.embedding, *self.blocks, self.final_norm, self.head]

    def tensor_specs(self) -> List[TensorSpec]:
        specs: List[TensorSpec] = []
        seen = set()
        for part in self.parts():
            for s in part.tensor_specs():
                if s.name in seen:
                    raise ValueError(f"two parts claim the tensor '{s.name}'")
                seen.add(s.name)
                specs.append(s)
        return specs

    def bind(self, tensors: Dict[str, torch.Tensor], dtype: torch.dtype) -> None:
        for part in self.parts():
            part.bind(tensors, dtype)

    def libraries(self, dtype: torch.dtype) -> List[str]:
        names: List[str] = []
        for part in self.parts():
            for lib in part.libraries(dtype):
                if lib not in names:
                    names.append(lib)
        return names

    def leaf_parts(self) -> List[Part]:
        """Every part of the model, the parts inside blocks (and inside those) included."""
        out: List[Part] = []

        def walk(part: Part) -> None:
            out.append(part)
            for child in part.children():
                walk(child)
        for part in self.parts():
            walk(part)
        return out

    def step_planners(self) -> Dict[Hashable, Part]:
        """One part per distinct ``step_plan_key``: the parts whose kernels want
        step metadata of their own (parts with equal keys share one plan)."""
        planners: Dict[Hashable, Part] = {}
        for part in self.leaf_parts():
            key = part.step_plan_key()
            if key is not None and key not in planners:
                planners[key] = part
        return planners

    def graph_capturable(self) -> bool:
        """Whether every part says that its forward pass may be recorded into a CUDA
        graph and replayed with new step metadata at the same addresses."""
        return all(part.graph_capturable for part in self.leaf_parts())

    # ---- cache -------------------------------------------------------------
    def cache_needs(self) -> List[Optional[CacheNeed]]:
        """Per stop of the schedule: what the cache manager keeps for it
        (``None`` for stops that keep nothing or read another stop's cache)."""
        needs: List[Optional[CacheNeed]] = []
        for stop in self.plan.schedule:
            need = self.blocks[stop.layer].mixer.cache_need() if stop.owns_cache else None
            needs.append(need)
        return needs

    # ---- forward ------------------------------------------------------------
    def forward(self, ctx: StepContext, caches: Sequence[CacheView],
                logit_rows: torch.Tensor, logits: torch.Tensor,
                all_rows_in_order: bool = False) -> torch.Tensor:
        """Run the step's tokens; write float32 logits of ``logit_rows`` into
        ``logits`` ``[len(logit_rows), vocab]``.  ``all_rows_in_order`` says
        that ``logit_rows`` is ``0..T-1``, which saves the row gather."""
        T = ctx.num_tokens
        H = self.plan.hidden_size
        residual = ctx.workspace.get("model.residual", (T, H), torch.float32)
        self.embedding.forward(ctx, residual)
        delta = None
        for stop, cache in zip(self.plan.schedule, caches):
            delta = self.blocks[stop.layer].forward(ctx, delta, residual, cache)
        n = logit_rows.numel()
        if n == 0:
            # caches are written; nobody asked for logits
            return logits
        x = self.final_norm.forward(ctx, delta, residual)
        if not all_rows_in_order:
            picked = ctx.workspace.get("model.picked", (n, H), ctx.dtype)
            ops.gather_rows(x, logit_rows, picked)
            x = picked
        self.head.forward(ctx, x, logits)
        return logits
