"""Interfaces of the parts a layer is put together from, and their registries.

A *part* is built from a :class:`PartSpec` (its ``kind`` picks the class, its
``params`` carry every size and constant), lists the tensors it needs, takes
them, and then runs on the tokens of a step.  No part knows which model it is
in: names of tensors, sizes and options all arrive as parameters.

Kinds of parts and what each must offer:

* **Norm**          ``forward(ctx, delta, residual) -> normed``.  Adds ``delta``
  (``[T, H]``, ``[T, k, H]`` or ``None``) into the float32 ``residual`` in place
  and returns the normalised rows in the activation dtype.
* **Position**      what a mixer applies to queries and keys: ``rotary_dim``,
  ``interleaved`` and ``table(device, positions)`` (``cos | sin`` per position).
* **Mixer**         ``cache_need()`` says what the cache manager must keep for
  it (pages of per-token data, a fixed-size state, or nothing);
  ``forward(ctx, x, cache) -> y`` mixes the tokens of each request in order.
* **FeedForward**   ``forward(ctx, x) -> y``, token by token.  ``y`` is ``[T, H]``
  or ``[T, k, H]``: k partial rows per token that the next norm adds in order.
* **Block**         arranges a mixer, a feed-forward (if it has one) and the
  norms it names around the residual stream:
  ``forward(ctx, delta, residual, cache) -> delta``.

Any part whose kernels want step metadata of their own (row lists, tile lists)
states a ``step_plan_key()`` and builds the lists in ``plan_step(shape)``; the
engine packs them into the step's one metadata copy and the part finds them
under ``ctx.plan(self)``.
* **Embedding / Head**  token ids -> residual rows; normed rows -> logits.

The reference wires the same roles by attribute walks over ``BaseOP`` objects
and a process-global context (python/freetoken/layers/base.py:15-53,
python/freetoken/core.py:112-207); here the context is an argument.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Dict, Hashable, List, Optional, Sequence, Tuple

import numpy as np
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


@dataclass
class StepShape:
    """The host-side facts of a step a part may plan from."""

    segments: List[Segment]
    num_tokens: int
    page_size: int
    table_width: int       # entries of a block-table row in this step
    max_q_len: int
    max_kv_len: int


@dataclass
class StepPlan:
    """Step metadata of one part (or of all parts with the same plan key):
    ``arrays`` are int32 lists that travel to the device with the step's metadata
    (afterwards found in ``tensors`` under the same names), ``host`` holds counts
    and sizes the part reads when it chooses and launches its kernels."""

    arrays: Dict[str, np.ndarray] = field(default_factory=dict)
    host: Dict[str, Any] = field(default_factory=dict)
    tensors: Dict[str, torch.Tensor] = field(default_factory=dict)


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
    # step metadata of the parts that plan their own, by plan key (the engine
    # fills this; a context made by hand gets a part's plan at its first use)
    plans: Dict[Hashable, StepPlan] = field(default_factory=dict)
    # when set, parts may leave measurements here (the benchmark counts the
    # experts a step touched); never set on the serving path
    probe: Optional[Dict[str, Any]] = None

    @property
    def num_segments(self) -> int:
        return len(self.segments)

    @property
    def decode_only(self) -> bool:
        return self.max_q_len == 1

    def shape(self) -> StepShape:
        width = self.block_tables[0].shape[1] if self.block_tables else 0
        return StepShape(self.segments, self.num_tokens, self.page_size, width, self.max_q_len,
                         self.max_kv_len)

    def plan(self, part: "Part") -> StepPlan:
        """The step metadata ``part`` planned.  The engine has it ready; for a
        context built by hand it is planned and copied to the device here."""
        key = part.step_plan_key()
        plan = self.plans.get(key)
        if plan is None:
            plan = part.plan_step(self.shape())
            for name, array in plan.arrays.items():
                plan.tensors[name] = torch.from_numpy(np.ascontiguousarray(array, dtype=np.int32)).to(self.device)
            self.plans[key] = plan
        return plan


@dataclass
class CacheView:
    """What one stop of the schedule sees of the cache."""

    # the stop's pages in the layout its need states (keys and values:
    # [2, pages, kv_heads, page, head_dim])
    kv_pages: Optional[torch.Tensor] = None
    block_table_index: int = 0                   # which entry of ctx.block_tables
    state: Optional[torch.Tensor] = None         # [slots + 1, *shape]
    writes: bool = True                          # False: reads another stop's cache

    @property
    def pages(self) -> Optional[torch.Tensor]:
        return self.kv_pages


# ------------------------------------------------------------------ parts
class Part:
    """Base of every part."""

    # A part that launches only work a CUDA graph can record - no host reads of
    # device data, and nothing that depends on the step's host-side lists
    # (``ctx.segments``) other than through sizes that a graph key fixes - says
    # so; decode steps of a model are replayed from a graph only if all its parts do.
    graph_capturable = False

    def __init__(self, spec: PartSpec, prefix: str):
        self.spec = spec
        self.prefix = prefix

    def children(self) -> List["Part"]:
        return []

    def step_plan_key(self) -> Optional[Hashable]:
        """``None``: the part needs no step metadata of its own.  Parts that
        return equal keys share one plan per step."""
        return None

    def plan_step(self, shape: StepShape) -> StepPlan:
        raise NotImplementedError

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
    """What a mixer may ask of a position encoding: how many leading dims of a
    head rotate (``rotary_dim``, 0: none), how they pair (``interleaved``:
    ``(2i, 2i+1)``, else halves ``(i, i + rotary_dim/2)``), and the table
    ``[>= positions, rotary_dim]`` of ``cos | sin`` per position in float32
    (``None`` when nothing rotates)."""

    rotary_dim: int = 0
    interleaved: bool = False

    def table(self, device, positions: int) -> Optional[torch.Tensor]:
        return None


class Mixer(Part):
    def cache_need(self) -> Optional[CacheNeed]:
        return None

    def forward(self, ctx: StepContext, x: torch.Tensor, cache: CacheView) -> torch.Tensor:
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, ctx: StepContext, x: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError


class Block(Part):
    """A mixer, a feed-forward (or none) and norms by name.  A block kind states
    the norms it arranges in ``NORM_NAMES`` and whether it has a feed-forward
    in ``HAS_FEED_FORWARD``; the model builds exactly those from the layer's spec."""

    NORM_NAMES: Tuple[str, ...] = ("mixer", "feed_forward")
    HAS_FEED_FORWARD = True

    def __init__(self, spec: PartSpec, prefix: str, mixer: Mixer, feed_forward: Optional[FeedForward],
                 norms: Dict[str, Norm]):
        super().__init__(spec, prefix)
        self.mixer = mixer
        self.feed_forward = feed_forward
        self.norms = dict(norms)

    @classmethod
    def check_parts(cls, prefix: str, norm_names: Sequence[str], has_feed_forward: bool) -> None:
        if sorted(norm_names) != sorted(cls.NORM_NAMES):
            raise ValueError(f"layer '{prefix}': a '{cls.__name__}' block arranges the norms "
                             f"{sorted(cls.NORM_NAMES)}, the layer lists {sorted(norm_names)}")
        if has_feed_forward != cls.HAS_FEED_FORWARD:
            raise ValueError(f"layer '{prefix}': a '{cls.__name__}' block "
                             f"{'needs' if cls.HAS_FEED_FORWARD else 'has no'} feed-forward")

    @property
    def mixer_norm(self) -> Norm:
        return self.norms["mixer"]

    @property
    def feed_forward_norm(self) -> Norm:
        return self.norms["feed_forward"]

    @property
    def graph_capturable(self) -> bool:       # a block records what its parts record
        return True

    def children(self) -> List[Part]:
        out: List[Part] = [self.mixer]
        if self.feed_forward is not None:
            out.append(self.feed_forward)
        return out + [self.norms[name] for name in sorted(self.norms)]

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
