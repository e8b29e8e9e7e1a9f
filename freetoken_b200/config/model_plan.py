"""Architecture-neutral description of a decoder: parts, layers, run order.

A model is data before it is code.  An architecture's typed configuration is
turned into a :class:`ModelPlan` that names, for every layer, which mixer,
feed-forward, norm and block arrangement to build and with which sizes; the
order in which layers run is a list of :class:`RunEntry`, which may name a
layer twice or let a layer read the cache another layer wrote.  Nothing below
this file knows which architecture it serves.

The reference reaches the same information through one generic ``ModelConfig``
with per-model payloads and ``attention_groups``
(python/freetoken/models/config.py:86-136,198-293); here it is explicit per layer.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Mapping, Optional, Tuple


@dataclass(frozen=True)
class PartSpec:
    """One part to build: a registry ``kind`` and its constructor parameters."""

    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)

    def get(self, key: str, default: Any = None) -> Any:
        return self.params.get(key, default)


@dataclass(frozen=True)
class LayerSpec:
    """The parts of one decoder layer and the block that arranges them.

    ``prefix`` is the tensor-name prefix of the layer's weights
    (``model.layers.3``); every part reads its tensors below it.  The block kind
    decides what a layer consists of: which norms it has (by the names the block
    knows them under) and whether it has a feed-forward at all.  The usual two
    norms have fields of their own (``mixer_norm`` is the norm named ``"mixer"``,
    ``feed_forward_norm`` the one named ``"feed_forward"``); any further norm of
    a block with more of them (post-norms, a sandwich) goes into ``norms``.
    """

    prefix: str
    block: PartSpec
    mixer: PartSpec
    feed_forward: Optional[PartSpec] = None
    mixer_norm: Optional[PartSpec] = None
    feed_forward_norm: Optional[PartSpec] = None
    norms: Mapping[str, PartSpec] = field(default_factory=dict)

    def all_norms(self) -> Dict[str, PartSpec]:
        """Every norm of the layer by name."""
        out: Dict[str, PartSpec] = {}
        if self.mixer_norm is not None:
            out["mixer"] = self.mixer_norm
        if self.feed_forward_norm is not None:
            out["feed_forward"] = self.feed_forward_norm
        for name, spec in self.norms.items():
            if name in out:
                raise ValueError(f"layer '{self.prefix}': the norm '{name}' is given twice")
            out[name] = spec
        return out


@dataclass(frozen=True)
class RunEntry:
    """One stop of the forward pass.

    ``layer`` indexes :attr:`ModelPlan.layers` (a layer named by two stops runs
    twice with the same weights).  Every stop has a cache of its own unless
    ``reads_cache_of`` names an earlier stop of the schedule: then the stop
    writes nothing and its mixer reads what that stop wrote.
    """

    layer: int
    reads_cache_of: Optional[int] = None

    @property
    def owns_cache(self) -> bool:
        return self.reads_cache_of is None


@dataclass(frozen=True)
class ModelPlan:
    """Everything the builder needs to put a model together."""

    architecture: str
    hidden_size: int
    vocab_size: int
    embedding: PartSpec
    layers: Tuple[LayerSpec, ...]
    schedule: Tuple[RunEntry, ...]
    final_norm: PartSpec
    head: PartSpec
    max_position: int

    def validate(self) -> None:
        n = len(self.layers)
        if n == 0:
            raise ValueError("a model plan needs at least one layer")
        if not self.schedule:
            raise ValueError("a model plan needs a schedule")
        for i, stop in enumerate(self.schedule):
            if not 0 <= stop.layer < n:
                raise ValueError(f"schedule[{i}] names layer {stop.layer}, outside 0..{n - 1}")
            src = stop.reads_cache_of
            if src is None:
                continue
            if not 0 <= src < i:
                raise ValueError(
                    f"schedule[{i}] reads the cache of stop {src}, which does not run before it"
                )
            if not self.schedule[src].owns_cache:
                raise ValueError(
                    f"schedule[{i}] reads the cache of stop {src}, which has no cache of its own"
                )

    def cache_owner(self, stop: int) -> int:
        """The stop whose cache ``stop`` uses (itself when it owns one)."""
        src = self.schedule[stop].reads_cache_of
        return stop if src is None else src


def sequential_schedule(num_layers: int) -> Tuple[RunEntry, ...]:
    """Layers 0..n-1, each once, each with a cache of its own."""
    return tuple(RunEntry(i) for i in range(num_layers))


def schedule_from_lists(
    order: List[int], reads_cache_of: Optional[Dict[int, int]] = None
) -> Tuple[RunEntry, ...]:
    """Build a schedule from a run order (layer indices) and an optional
    ``{stop: earlier stop}`` map of stops that read another stop's cache."""
    reads_cache_of = reads_cache_of or {}
    return tuple(RunEntry(layer, reads_cache_of.get(i)) for i, layer in enumerate(order))
