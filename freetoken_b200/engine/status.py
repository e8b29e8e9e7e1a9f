"""The scheduler's two throughput lines.

One line for every step that carries prompt tokens, one for every
``decode_log_interval``-th step that only decodes, with the wording of the
reference's reporter (python/freetoken/scheduler/status.py:79-123;
``decode_log_interval`` default 40, python/freetoken/scheduler/config.py:19).
A step here may mix prompt portions with decoded tokens; it is reported as a
prefill batch, its decoded tokens are still counted for the decode line.
"""

from __future__ import annotations

import time
from typing import Callable, Sequence


class StatusReporter:
    def __init__(self, log: Callable[[str], None], clock: Callable[[], float] = time.perf_counter,
                 decode_log_interval: int = 40):
        self.log = log
        self.clock = clock
        self.decode_log_interval = max(1, int(decode_log_interval))
        now = clock()
        self._last_prefill = now
        self._last_decode = now
        self._decode_steps = 0
        self._decoded = 0

    def report(self, plan: Sequence, *, running: int, queued: int, pages_used: int, pages_total: int,
               page_size: int) -> None:
        """``plan``: the step's planned entries (``tokens``, ``request`` each)."""
        usage = pages_used / pages_total if pages_total > 0 else 0.0
        new_tokens = sum(len(e.tokens) for e in plan if len(e.tokens) > 1)
        new_seqs = sum(1 for e in plan if len(e.tokens) > 1)
        self._decoded += sum(1 for e in plan if e.samples)
        now = self.clock()
        if new_tokens:
            gap = now - self._last_prefill
            self._last_prefill = now
            rate = new_tokens / gap if gap > 0 else 0.0
            self.log(f"Prefill batch, #new-seq: {new_seqs}, #new-token: {new_tokens}, #cached-token: 0, "
                     f"token usage: {usage:.2f}, #running-req: {running}, #queue-req: {queued}, "
                     f"input throughput (token/s): {rate:.2f}")
            return
        self._decode_steps += 1
        if self._decode_steps % self.decode_log_interval:
            return
        gap = now - self._last_decode
        self._last_decode = now
        rate = self._decoded / gap if gap > 0 else 0.0
        self._decoded = 0
        self.log(f"Decode batch, #running-req: {running}, #token: {pages_used * page_size}, "
                 f"token usage: {usage:.2f}, gen throughput (token/s): {rate:.2f}, #queue-req: {queued}")
