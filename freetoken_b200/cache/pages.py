"""Page accounting: a pool of fixed-size pages and who holds which.

The reference keeps a free list of page base offsets in a tensor, pops from
the front and appends on free, and checks ``free + cached == total`` when idle
(python/freetoken/scheduler/cache.py:35-38,533-571,608-632).  Here the free
list is a stack, so a page given back is the next one handed out (page reuse
shows up in tests after a handful of steps), and every page has exactly one
recorded state: free, or held by one owner.  Giving a page back twice, or a
page nobody holds, is an error at the call, not at the next audit.
"""

from __future__ import annotations

from typing import Dict, Hashable, Iterable, List


class OutOfPages(RuntimeError):
    """The pool has fewer free pages than were asked for."""


class PageAccountingError(RuntimeError):
    """A page was freed twice, freed by a stranger or lost."""


class PagePool:
    """``num_pages`` pages numbered ``first_page .. first_page+num_pages-1``.

    Pages below ``first_page`` are never handed out; page 0 is the sink that
    block-table entries of unused positions point at.
    """

    def __init__(self, num_pages: int, first_page: int = 1):
        if num_pages < 0:
            raise ValueError("num_pages must not be negative")
        self.num_pages = num_pages
        self.first_page = first_page
        # Stack: the lowest page number is handed out first, a freed page next.
        self._free: List[int] = list(range(first_page + num_pages - 1, first_page - 1, -1))
        self._holder: Dict[int, Hashable] = {}

    @property
    def free_pages(self) -> int:
        return len(self._free)

    @property
    def held_pages(self) -> int:
        return len(self._holder)

    def allocate(self, count: int, owner: Hashable) -> List[int]:
        if count < 0:
            raise ValueError("count must not be negative")
        if count > len(self._free):
            raise OutOfPages(f"asked for {count} pages, {len(self._free)} free of {self.num_pages}")
        pages = [self._free.pop() for _ in range(count)]
        for p in pages:
            self._holder[p] = owner
        return pages

    def release(self, pages: Iterable[int], owner: Hashable) -> None:
        pages = list(pages)
        for p in pages:
            holder = self._holder.get(p, _NOBODY)
            if holder is _NOBODY:
                raise PageAccountingError(f"page {p} is freed but nobody holds it")
            if holder != owner:
                raise PageAccountingError(f"page {p} is held by {holder!r}, freed by {owner!r}")
            del self._holder[p]
            self._free.append(p)

    def holder_of(self, page: int):
        return self._holder.get(page)

    def check(self) -> None:
        """Every page is free or held, exactly once."""
        free = set(self._free)
        if len(free) != len(self._free):
            raise PageAccountingError("a page is on the free list twice")
        held = set(self._holder)
        if free & held:
            raise PageAccountingError(f"pages both free and held: {sorted(free & held)[:8]}")
        everything = set(range(self.first_page, self.first_page + self.num_pages))
        if free | held != everything:
            lost = sorted(everything - free - held)
            raise PageAccountingError(f"pages lost: {lost[:8]}")


_NOBODY = object()
