"""What a part tells the loader about each tensor it needs.

A part lists :class:`TensorSpec` objects: the model-side name, the shape, how
the tensor is kept on the device (``role``), how the random-weights mode fills
it, and from which checkpoint tensors it may be assembled.  The reference
spreads the same knowledge over per-model ``iter_weights`` generators, merge
rules and attribute walks (python/freetoken/models/minimax_m3/weight.py:182-246,
python/freetoken/models/loader.py:17-21,110-133,265-289,
python/freetoken/layers/base.py:32-53).

Roles and the dtype a tensor has on the device:

* ``matrix``  - large tables and projection matrices.  A tensor stored in 16
  bits stays bfloat16 in both compute modes; one stored in 32 bits stays
  float32 in the float32 mode and is rounded to bfloat16 for the bfloat16 mode.
* ``small32`` - norm weights, router weights and biases: always float32 (the
  reference keeps the router's in float32 too, minimax_m3/moe.py:39-49).
* ``int32``   - integer tables.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import List, Tuple, Union

import torch

ROLES = ("matrix", "small32", "int32")


@dataclass(frozen=True)
class Name:
    """A checkpoint tensor taken as it is."""

    name: str
    shape: Tuple[int, ...]


@dataclass(frozen=True)
class Cat:
    """Checkpoint pieces joined along ``dim`` (q,k,v -> qkv; gate,up -> gate_up)."""

    parts: Tuple["Source", ...]
    dim: int = 0

    @property
    def shape(self) -> Tuple[int, ...]:
        first = list(self.parts[0].shape)
        first[self.dim] = sum(p.shape[self.dim] for p in self.parts)
        return tuple(first)


@dataclass(frozen=True)
class Stack:
    """Checkpoint pieces stacked along a new leading axis (one per expert)."""

    parts: Tuple["Source", ...]

    @property
    def shape(self) -> Tuple[int, ...]:
        return (len(self.parts),) + tuple(self.parts[0].shape)


Source = Union[Name, Cat, Stack]


def leaves(src: Source) -> List[Name]:
    if isinstance(src, Name):
        return [src]
    out: List[Name] = []
    for p in src.parts:
        out.extend(leaves(p))
    return out


def assemble(src: Source, read) -> torch.Tensor:
    """Build the tensor ``src`` describes; ``read(name)`` yields a leaf."""
    if isinstance(src, Name):
        return read(src.name)
    pieces = [assemble(p, read) for p in src.parts]
    if isinstance(src, Cat):
        return torch.cat(pieces, dim=src.dim)
    return torch.stack(pieces, dim=0)


def take_apart(src: Source, tensor: torch.Tensor, out: dict) -> None:
    """Inverse of :func:`assemble`: cut ``tensor`` into the leaves of ``src``."""
    if isinstance(src, Name):
        out[src.name] = tensor.contiguous()
        return
    if isinstance(src, Cat):
        sizes = [p.shape[src.dim] for p in src.parts]
        for p, piece in zip(src.parts, torch.split(tensor, sizes, dim=src.dim)):
            take_apart(p, piece, out)
        return
    for i, p in enumerate(src.parts):
        take_apart(p, tensor[i], out)


@dataclass(frozen=True)
class Init:
    """How the random-weights mode fills a tensor: ``mean + std * N(0,1)``."""

    mean: float = 0.0
    std: float = 0.02


@dataclass(frozen=True)
class TensorSpec:
    name: str
    shape: Tuple[int, ...]
    role: str = "matrix"
    init: Init = Init()
    # Ways to find the tensor in a checkpoint, tried in order.  Empty means
    # "by its own name".  The first entry is the layout the random-weights
    # mode writes.
    sources: Tuple[Source, ...] = ()
    # File dtype the random-weights mode uses for this tensor when the model
    # is written in 16 bits (router tensors stay float32 there).
    keep_float32_in_file: bool = False
    optional: bool = False
    # False: the tensor may be present in a checkpoint (it is checked like any
    # other) but is not loaded
    keep: bool = True
    # Which knob of the random-weights mode scales this tensor:
    # "matrix", "norm" or "router_bias".
    tag: str = "matrix"

    def __post_init__(self) -> None:
        if self.role not in ROLES:
            raise ValueError(f"tensor '{self.name}': unknown role {self.role!r}")

    def all_sources(self) -> Tuple[Source, ...]:
        own = Name(self.name, tuple(self.shape))
        if not self.sources:
            return (own,)
        if any(isinstance(s, Name) and s.name == self.name for s in self.sources):
            return self.sources
        return tuple(self.sources) + (own,)


def device_dtype(role: str, stored: torch.dtype, compute: torch.dtype) -> torch.dtype:
    """The dtype a tensor of ``role`` has on the device (see module docstring)."""
    if role == "small32":
        return torch.float32
    if role == "int32":
        return torch.int32
    if compute == torch.float32:
        return torch.bfloat16 if stored == torch.bfloat16 else torch.float32
    return torch.bfloat16
