"""The scheduler: admits requests, cuts prompts into portions, decodes, finishes.

Pure host logic over the :class:`CacheManager`; it never touches the device, so
its decisions are tested on the CPU with a stand-in for the model.

What the reference does and what is kept or changed:

* Queues: a FIFO of pending prompts with unfinished prompts at the front, and
  a set of running requests (python/freetoken/scheduler/prefill.py:232-301,
  decode.py:9-39).  Kept.
* Policy: the reference runs a prefill batch if anything is pending, else a
  decode batch (scheduler/scheduler.py:831-841).  Changed: every step carries
  one token of every running request AND prompt portions up to the token
  budget, since the step function takes mixed batches.
* Token budget: ``max_extend_tokens`` per batch, a prompt that does not fit is
  cut and continued first next time (prefill.py:125-126,159-162,263-285).  Kept
  as ``max_step_tokens``; decode tokens are charged first.
* Admission: a prompt is admitted if a request slot is free and its whole
  worst case (prompt + max_tokens) fits beside the worst case of everything
  already admitted (prefill.py:51-67, decode.py:27-30).  Kept, counted in
  pages per cache group.  So a running request never runs out of pages; WHEN
  PAGES RUN OUT, new requests wait in the queue, first come first served, until
  finished requests give pages back.  A request whose worst case exceeds the
  whole pool can never run and is refused when it is submitted.
* Finishing: ``length`` when ``max_tokens`` are out, ``stop`` on an EOS token
  unless ``ignore_eos``; EOS wins (scheduler.py:340-356,420-434).  A prompt at
  least as long as ``max_seq_len`` is refused and ``max_tokens`` is clamped to
  the room left (scheduler.py:492-523).  Kept.
"""

from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Hashable, Iterable, List, Optional, Sequence

from ..cache.manager import CacheManager
from ..sampling.params import SamplingParams


@dataclass
class Request:
    id: Hashable
    prompt: List[int]
    params: SamplingParams
    output: List[int] = field(default_factory=list)
    prompt_done: int = 0              # prompt tokens already run
    max_tokens: int = 0               # after clamping to the room left
    finish_reason: Optional[str] = None
    reserved: List[int] = field(default_factory=list)   # worst-case pages per group
    inflight: int = 0                 # sampling entries planned whose token is not yet recorded

    @property
    def finished(self) -> bool:
        return self.finish_reason is not None


@dataclass
class PlannedEntry:
    request: Request
    tokens: List[int]
    samples: bool          # True: the step's last token of this entry yields a new token
    from_device: bool = False   # the (single) input token is the one the previous step sampled,
                                # not yet read back: ``tokens`` holds a placeholder


class Scheduler:
    def __init__(self, cache: CacheManager, max_step_tokens: int = 8192,
                 eos_token_ids: Iterable[int] = (), detokenize=None):
        if max_step_tokens < 1:
            raise ValueError("max_step_tokens must be at least 1")
        self.cache = cache
        self.max_step_tokens = max_step_tokens
        self.eos = set(int(t) for t in eos_token_ids)
        self.detokenize = detokenize          # token ids -> text, for stop strings
        self.pending: Deque[Request] = deque()
        self.prefilling: Optional[Request] = None      # admitted, prompt not yet whole
        self.running: List[Request] = []               # decoding
        self.finished: List[Request] = []
        self._reserved = [0] * len(cache.paged_groups)

    # ---- submitting -------------------------------------------------------
    def submit(self, request: Request) -> bool:
        """Queue a request; ``False`` (with ``finish_reason`` set) if it can never run."""
        n = len(request.prompt)
        if n == 0:
            request.finish_reason = "rejected: empty prompt"
        elif n >= self.cache.max_seq_len:
            request.finish_reason = (f"rejected: prompt of {n} tokens does not fit "
                                     f"max_seq_len {self.cache.max_seq_len}")
        else:
            request.max_tokens = max(0, min(request.params.max_tokens, self.cache.max_seq_len - n))
            worst = self._worst_case(request)
            if any(w > t for w, t in zip(worst, self.cache.total_pages())):
                request.finish_reason = (f"rejected: needs {worst} pages, the pool has "
                                         f"{self.cache.total_pages()}")
            elif request.max_tokens == 0:
                request.finish_reason = "length"
        if request.finished:
            self.finished.append(request)
            return False
        self.pending.append(request)
        return True

    def _worst_case(self, request: Request) -> List[int]:
        total = len(request.prompt) + request.max_tokens
        return self.cache.worst_case_pages(total, self.max_step_tokens)

    # ---- planning a step ------------------------------------------------------
    def has_work(self) -> bool:
        return bool(self.pending or self.prefilling or self.running)

    def _admit(self, request: Request) -> bool:
        if self.cache.free_slots == 0:
            return False
        worst = self._worst_case(request)
        totals = self.cache.total_pages()
        if any(r + w > t for r, w, t in zip(self._reserved, worst, totals)):
            return False
        request.reserved = worst
        self._reserved = [r + w for r, w in zip(self._reserved, worst)]
        self.cache.admit(request.id)
        return True

    def plan(self) -> List[PlannedEntry]:
        """The next step's batch: one token per running request, then prompt
        portions in arrival order while budget, slots and pages last."""
        entries: List[PlannedEntry] = []
        for r in self.running:
            # A step may be planned while the one before it is still running
            # (its tokens not yet recorded): the request's input is then the token
            # on the device, and a request whose last token is among those in
            # flight gets no further step.  Whether it stopped on an EOS is only
            # known later; such a step's token is dropped by complete().
            if len(r.output) + r.inflight >= r.max_tokens:
                continue
            if r.inflight:
                entries.append(PlannedEntry(r, [0], True, True))
            else:
                entries.append(PlannedEntry(r, [r.output[-1]], True))
            r.inflight += 1
        budget = self.max_step_tokens - len(entries)
        while budget > 0:
            r = self.prefilling
            if r is None:
                if not self.pending or not self._admit(self.pending[0]):
                    break
                r = self.pending.popleft()
                self.prefilling = r
            take = min(budget, len(r.prompt) - r.prompt_done)
            whole = r.prompt_done + take == len(r.prompt)
            entries.append(PlannedEntry(r, r.prompt[r.prompt_done:r.prompt_done + take], whole))
            r.prompt_done += take           # progress is booked when planned
            budget -= take
            if not whole:
                break
            self.prefilling = None
            r.inflight += 1
            self.running.append(r)
        return entries

    # ---- after the step ----------------------------------------------------------
    def complete(self, entries: Sequence[PlannedEntry], sampled: Sequence[int]) -> List[Request]:
        """Record the step: ``sampled`` holds one token for every entry that
        samples, in order.  Returns the requests that finished."""
        done: List[Request] = []
        it = iter(sampled)
        for e in entries:
            r = e.request
            if not e.samples:
                continue
            token = int(next(it))
            r.inflight -= 1
            if r.finished:
                continue        # planned ahead before its EOS was read: the token is dropped
            r.output.append(token)
            if token in self.eos or token in r.params.stop_token_ids:
                if not r.params.ignore_eos:
                    r.finish_reason = "stop"
            if r.finish_reason is None and r.params.stop_strs and self._stop_str_shows(r):
                r.finish_reason = "stop"
            if r.finish_reason is None and len(r.output) >= r.max_tokens:
                r.finish_reason = "length"
            if r.finish_reason is not None:
                done.append(r)
        for r in done:
            self._retire(r)
        return done

    def _stop_str_shows(self, r: Request) -> bool:
        """Whether a stop string shows in the text of the newest tokens: a stop of
        N characters spans at most N tokens, so only that tail is decoded
        (python/freetoken/scheduler/scheduler.py:420-434)."""
        stops = [s for s in r.params.stop_strs if s]
        if not stops or self.detokenize is None:
            return False
        tail = r.output[-(max(len(s) for s in stops) + 1):]
        text = self.detokenize(tail)
        return any(s in text for s in stops)

    def _retire(self, r: Request) -> None:
        if r in self.running:
            self.running.remove(r)
        if self.cache.has_request(r.id):
            self.cache.release(r.id)
        self._reserved = [a - b for a, b in zip(self._reserved, r.reserved)]
        r.reserved = []
        self.finished.append(r)

    def abort(self, request_id: Hashable) -> bool:
        """Drop a request between steps; what it holds is given back."""
        for r in list(self.pending):
            if r.id == request_id:
                self.pending.remove(r)
                r.finish_reason = "abort"
                self.finished.append(r)
                return True
        if self.prefilling is not None and self.prefilling.id == request_id:
            r, self.prefilling = self.prefilling, None
            r.finish_reason = "abort"
            self._retire(r)
            return True
        for r in self.running:
            if r.id == request_id:
                r.finish_reason = "abort"
                self._retire(r)
                return True
        return False

    def check_integrity(self) -> None:
        self.cache.check_integrity()
        live = {r.id for r in self.running}
        if self.prefilling is not None:
            live.add(self.prefilling.id)
        if live != set(self.cache.live_requests()):
            raise AssertionError(f"scheduler holds {live}, the cache holds {set(self.cache.live_requests())}")
        want = [0] * len(self._reserved)
        for r in self.running + ([self.prefilling] if self.prefilling else []):
            want = [a + b for a, b in zip(want, r.reserved)]
        if want != self._reserved:
            raise AssertionError("page reservations do not add up")
