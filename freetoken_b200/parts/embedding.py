"""Token embedding and output head.

Embedding: ``residual[t,:] = W[ids[t],:]`` with no scale
(python/freetoken/layers/embedding.py:39-47, kernel/csrc/jit/index.cu:31-59).
Head: ``logits = x @ Wlm^T`` in float32 for the rows asked for; with tied
weights ``Wlm`` is the embedding table (layers/embedding.py:107-115).
"""

from __future__ import annotations

from typing import Dict, List

import torch

from ..csrc import ops
from ..weights.spec import TensorSpec
from . import linear
from .base import Embedding, Head, StepContext, register_embedding, register_head


@register_embedding("token_embedding")
class TokenEmbedding(Embedding):
    """params: ``vocab_size, hidden_size, scope``."""

    graph_capturable = True

    def __init__(self, spec, prefix):
        super().__init__(spec, prefix)
        self.vocab = int(spec.params["vocab_size"])
        self.hidden = int(spec.params["hidden_size"])
        self.weight_name = self.name(f"{spec.params['scope']}.weight")
        self.weight = None

    def tensor_specs(self) -> List[TensorSpec]:
        return [TensorSpec(self.weight_name, (self.vocab, self.hidden), tag="embedding")]

    def bind(self, tensors: Dict[str, torch.Tensor], dtype) -> None:
        self.weight = tensors[self.weight_name]

    def libraries(self, dtype) -> List[str]:
        return ["elementwise"]

    def forward(self, ctx: StepContext, residual: torch.Tensor) -> None:
        ops.embed_gather(ctx.token_ids, self.weight, residual)


@register_head("lm_head")
class LMHead(Head):
    """params: ``vocab_size, hidden_size, scope``, ``tied_to`` (full name of
    the embedding table, or None)."""

    graph_capturable = True

    def __init__(self, spec, prefix):
        super().__init__(spec, prefix)
        self.vocab = int(spec.params["vocab_size"])
        self.hidden = int(spec.params["hidden_size"])
        self.tied_to = spec.get("tied_to")
        self.own_name = self.name(f"{spec.params['scope']}.weight")
        self.weight_name = self.tied_to or self.own_name
        self.weight = None

    def tensor_specs(self) -> List[TensorSpec]:
        if self.tied_to:
            # a checkpoint of a tied model may still carry the head's tensor; it
            # is accepted and dropped (python/freetoken/layers/embedding.py:74-90)
            return [TensorSpec(self.own_name, (self.vocab, self.hidden), optional=True, keep=False)]
        return [TensorSpec(self.weight_name, (self.vocab, self.hidden))]

    def bind(self, tensors: Dict[str, torch.Tensor], dtype) -> None:
        self.weight = tensors[self.weight_name]

    def libraries(self, dtype) -> List[str]:
        return linear.libraries(dtype)

    def forward(self, ctx: StepContext, x: torch.Tensor, out: torch.Tensor) -> None:
        linear.linear(x, self.weight, out)
