"""Choosing next tokens from logits on the device.

Greedy is an argmax over the float32 logits; otherwise
``softmax(logits / T)``, the top-k and top-p filters a request asks for, and an
inverse-CDF draw with one uniform number per row
(python/freetoken/engine/sample.py:24-80; clamps ``T >= 1e-6``, ``top_p`` in
``[1e-6, 1]`` at :62-66).  The uniform comes from the request's own generator,
so a request's tokens are the same whatever else is in the batch.
"""

from __future__ import annotations

from typing import List, Optional, Sequence

import numpy as np
import torch

from ..csrc import ops
from .params import SamplingParams

MIN_T = 1e-6
MIN_P = 1e-6


class RequestRng:
    """One uniform in [0,1) per generated token, reproducible from a seed."""

    def __init__(self, seed: int):
        self._gen = torch.Generator(device="cpu")
        self._gen.manual_seed(int(seed) & ((1 << 63) - 1))

    def next_uniform(self) -> float:
        return float(torch.rand(1, generator=self._gen, dtype=torch.float64))


class Sampler:
    def __init__(self, device, vocab_size: int):
        self.device = torch.device(device)
        self.vocab_size = vocab_size
        self._probs: Optional[torch.Tensor] = None
        self._out: Optional[torch.Tensor] = None
        # per-row options travel through two pinned buffers taken in turn; a buffer
        # is written again only after the copy that last read it has finished
        self._pinned: List[Optional[torch.Tensor]] = [None, None]
        self._pinned_done: List[Optional[torch.cuda.Event]] = [None, None]
        self._options_dev: Optional[torch.Tensor] = None
        self._turn = 0

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams],
               uniforms: Sequence[float], out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``logits`` ``[rows, vocab]`` float32 on the device -> int32 ``[rows]`` there
        (in ``out`` if given, else in a buffer the next call overwrites)."""
        rows = logits.shape[0]
        if out is not None:
            out = out[:rows]
        else:
            if self._out is None or self._out.numel() < rows:
                self._out = torch.empty(max(rows, 64), dtype=torch.int32, device=self.device)
            out = self._out[:rows]
        if all(p.is_greedy for p in params):
            ops.sample(logits, None, None, None, None, out, None)
            return out
        V = logits.shape[1]
        turn = self._turn
        self._turn ^= 1
        cap = 0 if self._options_dev is None else self._options_dev.shape[1]
        if cap < rows:
            # larger batch than before: new buffers on both sides, [4, cap] each
            cap = max(rows, 64)
            torch.cuda.current_stream().synchronize()
            self._options_dev = torch.empty((4, cap), dtype=torch.float32, device=self.device)
            self._pinned = [torch.zeros((4, cap), dtype=torch.float32).pin_memory() for _ in range(2)]
            self._pinned_done = [torch.cuda.Event() for _ in range(2)]
        else:
            self._pinned_done[turn].synchronize()
        host = self._pinned[turn].numpy()
        for i, p in enumerate(params):
            host[0, i] = 0.0 if p.is_greedy else max(p.temperature, MIN_T)
            host[1, i] = min(max(p.top_p, MIN_P), 1.0)
            host[2, i] = min(max(uniforms[i], 0.0), 0.99999994)
        ks = np.asarray([p.top_k if 1 <= p.top_k < V else 0 for p in params], dtype=np.int32)
        host[3, :rows] = ks.view(np.float32)
        dev = self._options_dev
        dev.copy_(self._pinned[turn], non_blocking=True)
        self._pinned_done[turn].record()
        if self._probs is None or self._probs.numel() < rows * V:
            self._probs = torch.empty(rows * V, dtype=torch.float32, device=self.device)
        ops.sample(logits, dev[0, :rows], dev[3, :rows].view(torch.int32) if ks.any() else None,
                   dev[1, :rows] if (host[1, :rows] < 1.0).any() else None, dev[2, :rows], out,
                   self._probs)
        return out
