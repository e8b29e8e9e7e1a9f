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

from typing import Optional

import torch

from .base import Position, register_position


class _Rotary(Position):
    interleaved = False

    def __init__(self, spec, prefix):
        super().__init__(spec, prefix)
        self.head_dim = int(spec.params["head_dim"])
        self.rotary_dim = int(spec.params["rotary_dim"])
        self.theta = float(spec.params["theta"])
        self.max_position = int(spec.params["max_position"])
        if self.rotary_dim % 2 or not 0 <= self.rotary_dim <= self.head_dim:
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even and within head_dim {self.head_dim}")
        self._table: Optional[torch.Tensor] = None

    def table(self, device, positions: int) -> Optional[torch.Tensor]:
        """``[positions, rotary_dim]`` float32 on ``device`` (``None`` when nothing rotates)."""
        if self.rotary_dim == 0:
            return None
        positions = min(positions, self.max_position)
        if self._table is None or self._table.shape[0] < positions or self._table.device != torch.device(device):
            r = self.rotary_dim
            inv_freq = 1.0 / (self.theta ** (torch.arange(0, r, 2, dtype=torch.float) / r))
            t = torch.arange(positions, dtype=torch.float)
            freqs = torch.einsum("i,j -> ij", t, inv_freq)
            self._table = torch.cat((freqs.cos(), freqs.sin()), dim=-1).contiguous().to(device)
        return self._table


@register_position("rotary_neox")
class RotaryNeox(_Rotary):
    interleaved = False


@register_position("rotary_interleaved")
class RotaryInterleaved(_Rotary):
    interleaved = True


@register_position("none")
class NoPosition(Position):
    interleaved = False
    rotary_dim = 0

    def table(self, device, positions: int):
        return None
