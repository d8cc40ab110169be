"""Host-side bookkeeping of cache pages: which are free, which request holds which.

A page is either on the free list or held by exactly one request; giving back a page
that is not held, or holding one twice, is an error raised at once.  Free pages are
handed out last-in-first-out, so a page that was just given back is the next one used
(the reference's slot pool does the same with whole slots,
src/runtime/cache/cache_pool.cpp:86-126).
"""
from __future__ import annotations

from typing import Dict, List, Optional


class OutOfPages(RuntimeError):
    """No free page (or slot) is left for what was asked."""


class PageAccountingError(RuntimeError):
    """A page was given back twice, or by a request that does not hold it."""


class PagePool:
    def __init__(self, num_pages: int):
        if num_pages <= 0:
            raise ValueError("a page pool needs at least one page")
        self.num_pages = int(num_pages)
        self._free: List[int] = list(range(self.num_pages - 1, -1, -1))  # pop() hands out 0, 1, 2, ...
        self._owner: List[Optional[object]] = [None] * self.num_pages
        self.high_water = 0

    @property
    def n_free(self) -> int:
        return len(self._free)

    @property
    def n_held(self) -> int:
        return self.num_pages - len(self._free)

    def alloc(self, owner: object) -> int:
        if owner is None:
            raise ValueError("a page needs an owner")
        if not self._free:
            raise OutOfPages("no free page")
        page = self._free.pop()
        if self._owner[page] is not None:
            raise PageAccountingError(f"page {page} on the free list is held by {self._owner[page]!r}")
        self._owner[page] = owner
        self.high_water = max(self.high_water, self.n_held)
        return page

    def free(self, page: int, owner: object) -> None:
        if not 0 <= page < self.num_pages:
            raise PageAccountingError(f"page {page} does not exist")
        if self._owner[page] is None:
            raise PageAccountingError(f"page {page} is given back twice")
        if self._owner[page] != owner:
            raise PageAccountingError(f"page {page} is held by {self._owner[page]!r}, not {owner!r}")
        self._owner[page] = None
        self._free.append(page)

    def owner(self, page: int) -> Optional[object]:
        return self._owner[page]

    def check(self) -> None:
        """Raises unless every page is exactly once either free or held."""
        free = set(self._free)
        if len(free) != len(self._free):
            raise PageAccountingError("a page is on the free list twice")
        for p in range(self.num_pages):
            if (p in free) == (self._owner[p] is not None):
                raise PageAccountingError(f"page {p} is {'both free and held' if p in free else 'lost'}")
