"""Host-side page accounting: a free list of page ids with an owner per page.

The reference's page accountant keeps refcounts and throws when a reservation
cannot be met (runtime/kv_cache/paged_kv_cache.cpp:61-98).  This allocator is
all-or-nothing per call, refuses a page that is freed twice or by someone who does
not hold it, and hands back the most recently freed pages first, so that a page
is used again as soon as possible.
"""
from __future__ import annotations

from typing import Hashable, Iterable, List


class OutOfPages(RuntimeError):
    """A reservation needs more pages than are free.  Nothing was taken."""


class PageAccountingError(RuntimeError):
    """A page was freed twice, freed by a non-owner, or is out of range."""


class PageAllocator:
    def __init__(self, num_pages: int):
        if num_pages <= 0:
            raise ValueError(f"a page pool needs at least one page, got {num_pages}")
        self.num_pages = int(num_pages)
        self._free: List[int] = list(range(self.num_pages - 1, -1, -1))     # pop() gives 0, 1, 2, ...
        self._owner: List[Hashable] = [None] * self.num_pages
        self.allocations = 0            # pages handed out so far (reuse shows as allocations > num_pages)

    @property
    def num_free(self) -> int:
        return len(self._free)

    @property
    def num_used(self) -> int:
        return self.num_pages - len(self._free)

    def allocate(self, n: int, owner: Hashable) -> List[int]:
        if owner is None:
            raise ValueError("pages need an owner")
        if n < 0:
            raise ValueError(f"cannot allocate {n} pages")
        if n > len(self._free):
            raise OutOfPages(f"{n} pages wanted, {len(self._free)} of {self.num_pages} free")
        pages = [self._free.pop() for _ in range(n)]
        for p in pages:
            self._owner[p] = owner
        self.allocations += n
        return pages

    def release(self, pages: Iterable[int], owner: Hashable) -> None:
        pages = list(pages)
        for p in pages:                                   # check everything before changing anything
            if not 0 <= p < self.num_pages:
                raise PageAccountingError(f"page {p} is outside the pool of {self.num_pages}")
            if self._owner[p] is None:
                raise PageAccountingError(f"page {p} is freed twice")
            if self._owner[p] != owner:
                raise PageAccountingError(f"page {p} belongs to {self._owner[p]!r}, not to {owner!r}")
        if len(set(pages)) != len(pages):
            raise PageAccountingError(f"a page is named twice in one release: {pages}")
        for p in pages:
            self._owner[p] = None
            self._free.append(p)

    def owner_of(self, page: int):
        return self._owner[page]

    def check(self) -> None:
        """Every page is either free once or owned once."""
        free = set(self._free)
        if len(free) != len(self._free):
            raise PageAccountingError("a page is on the free list twice")
        for p in range(self.num_pages):
            if (p in free) == (self._owner[p] is not None):
                raise PageAccountingError(f"page {p}: free-list and owner table disagree")
