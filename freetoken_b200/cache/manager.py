"""The cache manager: request slots, block tables, page groups, state slots.

Host-side bookkeeping only; device memory lives in :mod:`.storage`.

What the reference does, and what is kept or changed:

* A request gets a row of a page table for its lifetime
  (python/freetoken/scheduler/table.py:4-30).  Kept: the *request slot* indexes
  the block table of every group and the per-request state slots.
* The page table holds a token slot per position
  (python/freetoken/core.py:170-171, scheduler/cache.py:634-667).  Changed: the
  block table holds one page number per ``page_size`` positions.
* Layers with different cache needs are described by group specs and each
  group is costed and pooled on its own
  (python/freetoken/models/config.py:86-110, kvcache/base.py:19-32).  Kept:
  mixers state a :class:`CacheNeed`; equal needs share a :class:`PageGroup`
  with pages of its own.  A group with a window gives pages back while the
  request runs, once the window has passed them (scheduler/cache.py:171-231).
* Pages are allocated for exactly the tokens a step writes
  (scheduler/cache.py:256-275) and go back when the request ends
  (scheduler/cache.py:512-519).  Kept.
* Fixed-size per-request state lives in slots indexed like the request
  (python/freetoken/kvcache/linear_state_pool.py:32-78).  Kept as
  :class:`StateNeed` groups; the slot is cleared when a request is admitted.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Hashable, List, Optional, Sequence, Tuple

import numpy as np

from .pages import OutOfPages, PageAccountingError, PagePool


class PerTokenNeed:
    """Base of needs that keep something for every token of a request, in
    pages.  A need states the layout of its pages and what a token costs; the
    manager pools stops with equal needs, the storage allocates
    ``[stops, *layout(pages, page_size)]`` per group.  ``window`` = how many
    latest tokens are still read (``None``: all of them): pages the window has
    passed are given back while the request runs.  ``storage_dtype`` names the
    element type (``None``: the engine's activation dtype).

    A cache of another shape per token (one latent vector instead of keys and
    values, keys and values of different widths) is another subclass; nothing in
    the manager, the storage or the engine names a particular one."""

    kind = "per_token"
    window: Optional[int] = None
    storage_dtype: Optional[str] = None
    page_axis = 0            # which axis of ``layout`` counts pages

    def layout(self, pages: int, page_size: int) -> Tuple[int, ...]:
        raise NotImplementedError

    def elements_per_token(self) -> int:
        raise NotImplementedError


class PerRequestNeed:
    """Base of needs that keep a tensor of fixed ``shape`` per request, carried
    from step to step in the request's slot and cleared when it is admitted."""

    kind = "per_request"
    shape: Tuple[int, ...] = ()
    dtype: str = "float32"


@dataclass(frozen=True)
class PagedKVNeed(PerTokenNeed):
    """Keys and values per token; ``window`` = how many latest keys are read
    (``None``: all of them).  Pages are ``[2 (K, V), pages, kv_heads, page_size,
    head_dim]``: a page of one KV head is ``page_size * head_dim`` contiguous
    elements, the tile the attention kernels stream."""

    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None
    kind: str = "paged_kv"
    page_axis = 1

    def layout(self, pages: int, page_size: int) -> Tuple[int, ...]:
        return (2, pages, self.num_kv_heads, page_size, self.head_dim)

    def elements_per_token(self) -> int:
        return 2 * self.num_kv_heads * self.head_dim


@dataclass(frozen=True)
class StateNeed(PerRequestNeed):
    """A tensor of fixed ``shape`` per request, carried from step to step."""

    shape: Tuple[int, ...]
    dtype: str = "float32"
    kind: str = "state"


CacheNeed = PerTokenNeed | PerRequestNeed


@dataclass
class PageGroup:
    """Stops with the same paged need: own pool, own block table."""

    need: PerTokenNeed
    stops: List[int]
    pool: PagePool
    block_table: np.ndarray  # int32 [max_slots, max_pages_per_request], 0 = sink page
    # first page index still held, per slot (pages below it were given back)
    first_held: np.ndarray   # int32 [max_slots]
    # number of table entries ever filled, per slot
    filled: np.ndarray       # int32 [max_slots]


@dataclass
class StateGroup:
    need: PerRequestNeed
    stops: List[int]


class NoFreeSlot(RuntimeError):
    """All request slots are taken."""


class CacheManager:
    """Slots, block tables and pages for up to ``max_slots`` live requests."""

    def __init__(self, needs: Sequence[Optional[CacheNeed]], page_size: int,
                 num_pages: int | Sequence[int], max_slots: int, max_seq_len: int):
        """``needs[i]`` is the need of the i-th cache-owning stop of the
        schedule (``None``: that stop keeps nothing).  ``num_pages`` is the
        pool size of every paged group, or one size per group in order of
        first appearance."""
        if page_size <= 0:
            raise ValueError("page_size must be positive")
        self.page_size = page_size
        self.max_slots = max_slots
        self.max_seq_len = max_seq_len
        self.max_pages_per_request = -(-max_seq_len // page_size)
        self.paged_groups: List[PageGroup] = []
        self.state_groups: List[StateGroup] = []
        # stop -> (group index, index of the stop inside the group)
        self.paged_index: Dict[int, Tuple[int, int]] = {}
        self.state_index: Dict[int, Tuple[int, int]] = {}
        paged_needs: List[PerTokenNeed] = []
        for stop, need in enumerate(needs):
            if need is None:
                continue
            if isinstance(need, PerTokenNeed):
                if need not in paged_needs:
                    paged_needs.append(need)
                    g = len(paged_needs) - 1
                    pages = num_pages if isinstance(num_pages, int) else num_pages[g]
                    self.paged_groups.append(PageGroup(
                        need=need, stops=[], pool=PagePool(pages),
                        block_table=np.zeros((max_slots, self.max_pages_per_request), np.int32),
                        first_held=np.zeros(max_slots, np.int32),
                        filled=np.zeros(max_slots, np.int32),
                    ))
                g = paged_needs.index(need)
                self.paged_index[stop] = (g, len(self.paged_groups[g].stops))
                self.paged_groups[g].stops.append(stop)
            elif isinstance(need, PerRequestNeed):
                for g, group in enumerate(self.state_groups):
                    if group.need == need:
                        break
                else:
                    self.state_groups.append(StateGroup(need, []))
                    g = len(self.state_groups) - 1
                self.state_index[stop] = (g, len(self.state_groups[g].stops))
                self.state_groups[g].stops.append(stop)
            else:
                raise ValueError(f"stop {stop}: a cache need is a PerTokenNeed or a PerRequestNeed, "
                                 f"not {need!r}")
        self._free_slots: List[int] = list(range(max_slots - 1, -1, -1))
        self._slot_of: Dict[Hashable, int] = {}
        self._request_of: Dict[int, Hashable] = {}
        self.seq_len = np.zeros(max_slots, np.int64)
        # slots admitted since the last call of take_fresh_slots(): their
        # state rows have to be cleared on the device before they are used
        self._fresh: List[int] = []
        # pages given back, kept for take_freed() when record_freed is set
        self.record_freed = False
        self._freed: List[Tuple[int, List[int]]] = []

    # ---- request slots --------------------------------------------------
    @property
    def free_slots(self) -> int:
        return len(self._free_slots)

    def has_request(self, request: Hashable) -> bool:
        return request in self._slot_of

    def slot(self, request: Hashable) -> int:
        return self._slot_of[request]

    def live_requests(self) -> List[Hashable]:
        return list(self._slot_of)

    def length(self, request: Hashable) -> int:
        return int(self.seq_len[self._slot_of[request]])

    def admit(self, request: Hashable) -> int:
        if request in self._slot_of:
            raise ValueError(f"request {request!r} is already live")
        if not self._free_slots:
            raise NoFreeSlot(f"all {self.max_slots} request slots are taken")
        slot = self._free_slots.pop()
        self._slot_of[request] = slot
        self._request_of[slot] = request
        self.seq_len[slot] = 0
        for group in self.paged_groups:
            group.block_table[slot, :] = 0
            group.first_held[slot] = 0
            group.filled[slot] = 0
        self._fresh.append(slot)
        return slot

    def take_fresh_slots(self) -> List[int]:
        fresh, self._fresh = self._fresh, []
        return fresh

    # ---- pages ------------------------------------------------------------
    def _pages_for(self, length: int) -> int:
        return -(-length // self.page_size)

    def pages_to_grow(self, request: Hashable, new_len: int) -> List[int]:
        """Pages each group must allocate so the request can reach ``new_len``."""
        slot = self._slot_of[request]
        return [max(0, self._pages_for(new_len) - int(g.filled[slot])) for g in self.paged_groups]

    def can_grow(self, request: Hashable, new_len: int) -> bool:
        need = self.pages_to_grow(request, new_len)
        return all(n <= g.pool.free_pages for n, g in zip(need, self.paged_groups))

    def grow(self, request: Hashable, new_len: int) -> None:
        """Make every position below ``new_len`` addressable in every group.

        Either all groups get their pages or none does."""
        slot = self._slot_of[request]
        if new_len > self.max_seq_len:
            raise ValueError(f"request {request!r}: length {new_len} exceeds max_seq_len {self.max_seq_len}")
        need = self.pages_to_grow(request, new_len)
        for n, g in zip(need, self.paged_groups):
            if n > g.pool.free_pages:
                raise OutOfPages(
                    f"request {request!r} needs {n} more pages to reach {new_len} tokens, "
                    f"{g.pool.free_pages} free of {g.pool.num_pages}")
        for n, g in zip(need, self.paged_groups):
            if n == 0:
                continue
            start = int(g.filled[slot])
            g.block_table[slot, start:start + n] = g.pool.allocate(n, (request, id(g)))
            g.filled[slot] = start + n

    def advance(self, request: Hashable, n_tokens: int) -> None:
        """Record that ``n_tokens`` more tokens were written; windows that
        have passed whole pages give them back."""
        slot = self._slot_of[request]
        new_len = int(self.seq_len[slot]) + n_tokens
        for g in self.paged_groups:
            if new_len > int(g.filled[slot]) * self.page_size:
                raise PageAccountingError(
                    f"request {request!r} advanced to {new_len} tokens without pages for them")
        self.seq_len[slot] = new_len
        for g in self.paged_groups:
            w = g.need.window
            if w is None:
                continue
            # The next query sits at position new_len and reads keys
            # new_len-w+1 .. new_len; pages wholly below that are dead.
            dead_below = max(0, new_len - w + 1) // self.page_size
            first = int(g.first_held[slot])
            if dead_below > first:
                self._note_freed(g, g.block_table[slot, first:dead_below].tolist())
                g.pool.release(g.block_table[slot, first:dead_below].tolist(), (request, id(g)))
                g.block_table[slot, first:dead_below] = 0
                g.first_held[slot] = dead_below

    def _note_freed(self, group, pages: List[int]) -> None:
        if self.record_freed and pages:
            self._freed.append((self.paged_groups.index(group), list(pages)))

    def take_freed(self) -> List[Tuple[int, List[int]]]:
        """``(group index, pages)`` given back since the last call (only kept
        when ``record_freed`` is set: a debugging aid that lets the engine
        overwrite freed pages, so that a read of stale data shows)."""
        out, self._freed = self._freed, []
        return out

    def release(self, request: Hashable) -> None:
        """The request is over: pages and slot go back at once."""
        slot = self._slot_of.pop(request)
        del self._request_of[slot]
        for g in self.paged_groups:
            first, filled = int(g.first_held[slot]), int(g.filled[slot])
            self._note_freed(g, g.block_table[slot, first:filled].tolist())
            g.pool.release(g.block_table[slot, first:filled].tolist(), (request, id(g)))
            g.block_table[slot, :] = 0
            g.first_held[slot] = 0
            g.filled[slot] = 0
        self.seq_len[slot] = 0
        if slot in self._fresh:
            self._fresh.remove(slot)
        self._free_slots.append(slot)

    # ---- planning help for the scheduler -------------------------------
    def worst_case_pages(self, total_len: int, largest_step: int) -> List[int]:
        """Most pages a request of ``total_len`` tokens ever holds per group
        when no step brings more than ``largest_step`` tokens."""
        out = []
        for g in self.paged_groups:
            full = self._pages_for(total_len)
            w = g.need.window
            if w is None:
                out.append(full)
            else:
                # live span: window + the step's tokens, not page aligned
                span = w + largest_step
                out.append(min(full, span // self.page_size + 2))
        return out

    def total_pages(self) -> List[int]:
        return [g.pool.num_pages for g in self.paged_groups]

    def free_pages(self) -> List[int]:
        return [g.pool.free_pages for g in self.paged_groups]

    def held_pages(self, request: Hashable) -> List[int]:
        slot = self._slot_of[request]
        return [int(g.filled[slot]) - int(g.first_held[slot]) for g in self.paged_groups]

    # ---- audit ---------------------------------------------------------------
    def check_integrity(self) -> None:
        """No page lost, held twice or free while in a block table."""
        live_slots = set(self._slot_of.values())
        if len(live_slots) != len(self._slot_of):
            raise PageAccountingError("two requests share a slot")
        if live_slots & set(self._free_slots) or len(live_slots) + len(self._free_slots) != self.max_slots:
            raise PageAccountingError("request slots do not add up")
        for g in self.paged_groups:
            g.pool.check()
            seen: Dict[int, int] = {}
            for slot in range(self.max_slots):
                first, filled = int(g.first_held[slot]), int(g.filled[slot])
                row = g.block_table[slot]
                if slot not in live_slots:
                    if filled or row.any():
                        raise PageAccountingError(f"free slot {slot} still has block-table entries")
                    continue
                if row[:first].any() or row[filled:].any():
                    raise PageAccountingError(f"slot {slot}: entries outside the held range")
                for p in row[first:filled].tolist():
                    if p < g.pool.first_page:
                        raise PageAccountingError(f"slot {slot}: held range points at the sink page")
                    if p in seen:
                        raise PageAccountingError(f"page {p} is in the tables of slots {seen[p]} and {slot}")
                    seen[p] = slot
                    if g.pool.holder_of(p) != (self._request_of[slot], id(g)):
                        raise PageAccountingError(f"page {p} in slot {slot}'s table is not held by its request")
            if len(seen) != g.pool.held_pages:
                raise PageAccountingError(
                    f"{g.pool.held_pages} pages are held but {len(seen)} are in block tables")
