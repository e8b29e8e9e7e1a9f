"""Position encodings a mixer applies to queries and keys.

Rotary: ``inv_freq_i = theta^(-2i/R)``, ``cos_sin[p] = [cos(p*inv_freq) |
sin(p*inv_freq)]`` in float32 over the first ``R = rotary_dim`` dims of every
head, the rest untouched (python/freetoken/layers/rotary.py:40-59).  Pairing is
NeoX halves ``(i, i+R/2)`` or interleaved ``(2i, 2i+1)``
(python/freetoken/kernel/triton/rope.py:62-78).  The table is computed on the
host in float32, as the reference computes it, and cut to the positions the
engine can reach.  ``none`` rotates nothing.
"""

from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from .base import Position, register_position

# One cos|sin table per (rotary_dim, theta, device), shared by every layer that
# rotates the same way (the reference shares one module through a cached
# ``get_rope``, python/freetoken/layers/rotary.py:212-213).  A table only grows.
_TABLES: Dict[Tuple[int, float, torch.device], torch.Tensor] = {}


def rotary_table(rotary_dim: int, theta: float, device, positions: int) -> torch.Tensor:
    """``[>= positions, rotary_dim]`` float32 on ``device``: ``cos | sin`` of
    ``position * theta^(-2i/rotary_dim)``, computed on the host in float32."""
    key = (int(rotary_dim), float(theta), torch.device(device))
    table = _TABLES.get(key)
    if table is None or table.shape[0] < positions:
        r = int(rotary_dim)
        inv_freq = 1.0 / (float(theta) ** (torch.arange(0, r, 2, dtype=torch.float) / r))
        t = torch.arange(positions, dtype=torch.float)
        freqs = torch.einsum("i,j -> ij", t, inv_freq)
        table = torch.cat((freqs.cos(), freqs.sin()), dim=-1).contiguous().to(device)
        _TABLES[key] = table
    return table


class _Rotary(Position):
    graph_capturable = True
    interleaved = False

    def __init__(self, spec, prefix):
        super().__init__(spec, prefix)
        self.head_dim = int(spec.params["head_dim"])
        self.rotary_dim = int(spec.params["rotary_dim"])
        self.theta = float(spec.params["theta"])
        self.max_position = int(spec.params["max_position"])
        if self.rotary_dim % 2 or not 0 <= self.rotary_dim <= self.head_dim:
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even and within head_dim {self.head_dim}")

    def table(self, device, positions: int) -> Optional[torch.Tensor]:
        """``[>= positions, rotary_dim]`` float32 on ``device`` (``None`` when
        nothing rotates); every layer with the same rotation gets the same tensor."""
        if self.rotary_dim == 0:
            return None
        return rotary_table(self.rotary_dim, self.theta, device, min(positions, self.max_position))


@register_position("rotary_neox")
class RotaryNeox(_Rotary):
    interleaved = False


@register_position("rotary_interleaved")
class RotaryInterleaved(_Rotary):
    interleaved = True


@register_position("none")
class NoPosition(Position):
    graph_capturable = True
    interleaved = False
    rotary_dim = 0

    def table(self, device, positions: int):
        return None
