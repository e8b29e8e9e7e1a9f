"""Interfaces of the parts a layer is put together from, and their registries.

A *part* is built from a :class:`PartSpec` (its ``kind`` picks the class, its
``params`` carry every size and constant), lists the tensors it needs, takes
them, and then runs on the tokens of a step.  No part knows which model it is
in: names of tensors, sizes and options all arrive as parameters.

Kinds of parts and what each must offer:

* **Norm**          ``forward(ctx, delta, residual) -> normed``.  Adds ``delta``
  (``[T, H]``, ``[T, k, H]`` or ``None``) into the float32 ``residual`` in place
  and returns the normalised rows in the activation dtype.
* **Position**      tables or constants a mixer applies to queries and keys.
* **Mixer**         ``cache_need()`` says what the cache manager must keep for
  it (paged keys/values, a fixed-size state, or nothing);
  ``forward(ctx, x, cache) -> y`` mixes the tokens of each request in order.
* **FeedForward**   ``forward(ctx, x) -> y``, token by token.  ``y`` is ``[T, H]``
  or ``[T, k, H]``: k partial rows per token that the next norm adds in order.
* **Block**         arranges a mixer, a feed-forward and their norms around the
  residual stream: ``forward(ctx, delta, residual, cache) -> delta``.
* **Embedding / Head**  token ids -> residual rows; normed rows -> logits.

The reference wires the same roles by attribute walks over ``BaseOP`` objects
and a process-global context (python/freetoken/layers/base.py:15-53,
python/freetoken/core.py:112-207); here the context is an argument.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple

import torch

from ..cache.manager import CacheNeed
from ..config.model_plan import PartSpec
from ..weights.spec import TensorSpec


# --------------------------------------------------------------- context
@dataclass
class Segment:
    """The tokens one request brings to a step: ``n`` tokens starting at
    position ``pos0`` of request slot ``slot``; rows ``q_start .. q_start+n-1``
    of the step's flat token list."""

    slot: int
    pos0: int
    n: int
    q_start: int


class Workspace:
    """Named scratch tensors that persist from step to step.

    ``get`` returns a view of a buffer at least as large as asked; a buffer is
    only ever replaced by a larger one, so steady-state steps allocate
    nothing."""

    def __init__(self, device):
        self.device = torch.device(device)
        self._buffers: Dict[str, torch.Tensor] = {}
        # bumped whenever a buffer is (re)allocated: captured CUDA graphs hold
        # raw addresses and must be dropped then
        self.generation = 0

    def get(self, name: str, shape: Sequence[int], dtype: torch.dtype) -> torch.Tensor:
        count = 1
        for s in shape:
            count *= int(s)
        buf = self._buffers.get(name)
        if buf is None or buf.dtype != dtype or buf.numel() < count:
            grow = max(count, 1)
            buf = torch.empty(grow, dtype=dtype, device=self.device)
            self._buffers[name] = buf
            self.generation += 1
        return buf[:count].view(*shape)

    def bytes(self) -> int:
        return sum(b.numel() * b.element_size() for b in self._buffers.values())


PREFILL_TILE = 64   # query tokens per tile of the prefill attention kernel


@dataclass
class StepContext:
    """Everything a part may read about the step it runs in."""

    device: torch.device
    dtype: torch.dtype                 # activation dtype: float32 or bfloat16
    segments: List[Segment]            # host copy, in batch order
    num_tokens: int
    # device int32 tensors
    token_ids: torch.Tensor            # [T]
    token_pos: torch.Tensor            # [T] absolute position of each token
    token_seg: torch.Tensor            # [T] index into segments
    seg_slot: torch.Tensor             # [S]
    seg_pos0: torch.Tensor             # [S]
    seg_q_start: torch.Tensor          # [S+1]
    seg_kv_len: torch.Tensor           # [S] pos0 + n
    block_tables: List[torch.Tensor]   # per page group: [S, width] page ids of the segments
    workspace: Workspace
    page_size: int
    # host-side summaries for kernel choice
    max_q_len: int = 1
    max_kv_len: int = 1
    max_positions: int = 0             # longest sequence the engine can hold
    # token rows of single-token segments (decode) and of longer segments, as
    # device int32 tensors; None when the step has none of that kind
    decode_rows: Optional[torch.Tensor] = None
    prefill_rows: Optional[torch.Tensor] = None
    num_decode_rows: int = 0
    num_prefill_rows: int = 0
    max_decode_kv_len: int = 0
    # query tiles (PREFILL_TILE tokens) of the longer segments: segment index
    # and first token inside the segment, device int32
    prefill_tile_seg: Optional[torch.Tensor] = None
    prefill_tile_q0: Optional[torch.Tensor] = None
    num_prefill_tiles: int = 0
    # query-key pairs the longer segments score (n * (pos0 + n/2), summed)
    prefill_scores: int = 0
    # when set, parts may leave measurements here (the benchmark counts the
    # experts a step touched); never set on the serving path
    probe: Optional[Dict[str, Any]] = None

    @property
    def num_segments(self) -> int:
        return len(self.segments)

    @property
    def decode_only(self) -> bool:
        return self.max_q_len == 1


@dataclass
class CacheView:
    """What one stop of the schedule sees of the cache."""

    kv_pages: Optional[torch.Tensor] = None     # [2, pages, kv_heads, page, head_dim]
    block_table_index: int = 0                   # which entry of ctx.block_tables
    state: Optional[torch.Tensor] = None         # [slots + 1, *shape]
    writes: bool = True                          # False: reads another stop's cache


# ------------------------------------------------------------------ parts
class Part:
    """Base of every part."""

    def __init__(self, spec: PartSpec, prefix: str):
        self.spec = spec
        self.prefix = prefix

    def name(self, local: str) -> str:
        return f"{self.prefix}.{local}" if self.prefix else local

    def tensor_specs(self) -> List[TensorSpec]:
        return []

    def bind(self, tensors: Dict[str, torch.Tensor], dtype: torch.dtype) -> None:
        """Take this part's tensors out of ``tensors`` (by full name)."""

    def libraries(self, dtype: torch.dtype) -> List[str]:
        """CUDA libraries this part launches for compute dtype ``dtype``."""
        return []


class Norm(Part):
    def forward(self, ctx: StepContext, delta: Optional[torch.Tensor],
                residual: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError


class Position(Part):
    pass


class Mixer(Part):
    def cache_need(self) -> Optional[CacheNeed]:
        return None

    def forward(self, ctx: StepContext, x: torch.Tensor, cache: CacheView) -> torch.Tensor:
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, ctx: StepContext, x: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError


class Block(Part):
    def __init__(self, spec: PartSpec, prefix: str, mixer: Mixer, feed_forward: FeedForward,
                 mixer_norm: Norm, feed_forward_norm: Norm):
        super().__init__(spec, prefix)
        self.mixer = mixer
        self.feed_forward = feed_forward
        self.mixer_norm = mixer_norm
        self.feed_forward_norm = feed_forward_norm

    def children(self) -> List[Part]:
        return [self.mixer, self.feed_forward, self.mixer_norm, self.feed_forward_norm]

    def tensor_specs(self) -> List[TensorSpec]:
        out: List[TensorSpec] = []
        for c in self.children():
            out.extend(c.tensor_specs())
        return out

    def bind(self, tensors, dtype) -> None:
        for c in self.children():
            c.bind(tensors, dtype)

    def libraries(self, dtype) -> List[str]:
        out: List[str] = []
        for c in self.children():
            out.extend(c.libraries(dtype))
        return out

    def forward(self, ctx: StepContext, delta: Optional[torch.Tensor], residual: torch.Tensor,
                cache: CacheView) -> torch.Tensor:
        raise NotImplementedError


class Embedding(Part):
    def forward(self, ctx: StepContext, residual: torch.Tensor) -> None:
        raise NotImplementedError


class Head(Part):
    def forward(self, ctx: StepContext, x: torch.Tensor, out: torch.Tensor) -> None:
        raise NotImplementedError


# ------------------------------------------------------------- registries
class Registry:
    """``kind`` -> class, per role."""

    def __init__(self, role: str):
        self.role = role
        self._classes: Dict[str, type] = {}

    def register(self, kind: str) -> Callable[[type], type]:
        def wrap(cls: type) -> type:
            self._classes[kind] = cls
            return cls
        return wrap

    def get(self, kind: str) -> type:
        try:
            return self._classes[kind]
        except KeyError:
            known = ", ".join(sorted(self._classes)) or "none"
            raise KeyError(f"no {self.role} of kind '{kind}' is registered (known: {known})") from None

    def kinds(self) -> List[str]:
        return sorted(self._classes)


NORMS = Registry("norm")
POSITIONS = Registry("position encoding")
MIXERS = Registry("mixer")
FEED_FORWARDS = Registry("feed-forward")
BLOCKS = Registry("block")
EMBEDDINGS = Registry("embedding")
HEADS = Registry("head")

register_norm = NORMS.register
register_position = POSITIONS.register
register_mixer = MIXERS.register
register_feed_forward = FEED_FORWARDS.register
register_block = BLOCKS.register
register_embedding = EMBEDDINGS.register
register_head = HEADS.register
