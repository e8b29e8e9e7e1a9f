"""RMSNorm with the residual add folded in.

``z = delta + residual; residual <- z; y = z * rsqrt(mean(z^2) + eps) * w``
in float32 (python/freetoken/kernel/triton/norm.py:101-112); ``plus_one``
selects the ``(1 + w)`` form (norm.py:69-72, python/freetoken/layers/norm.py:120-147).
The residual stream itself stays float32 between layers here (the reference
rounds it to the activation dtype each time it is stored, norm.py:108-109).
"""

from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..csrc import ops
from ..weights.spec import Init, TensorSpec
from .base import Norm, StepContext, register_norm


@register_norm("rmsnorm")
class RMSNorm(Norm):
    """params: ``size``, ``eps``, ``plus_one``, ``scope`` (tensor name below the prefix)."""

    graph_capturable = True

    def __init__(self, spec, prefix):
        super().__init__(spec, prefix)
        self.size = int(spec.params["size"])
        self.eps = float(spec.params["eps"])
        self.plus_one = bool(spec.get("plus_one", False))
        self.weight_name = self.name(f"{spec.params['scope']}.weight")
        self.weight: Optional[torch.Tensor] = None

    def tensor_specs(self) -> List[TensorSpec]:
        mean = 0.0 if self.plus_one else 1.0
        return [TensorSpec(self.weight_name, (self.size,), role="small32",
                           init=Init(mean=mean, std=0.0), tag="norm")]

    def bind(self, tensors: Dict[str, torch.Tensor], dtype) -> None:
        self.weight = tensors[self.weight_name]

    def libraries(self, dtype) -> List[str]:
        return ["elementwise"]

    def forward(self, ctx: StepContext, delta, residual: torch.Tensor) -> torch.Tensor:
        out = ctx.workspace.get("norm.out", residual.shape, ctx.dtype)
        ops.rmsnorm(delta, residual, self.weight, out, self.eps, self.plus_one)
        return out
