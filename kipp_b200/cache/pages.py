"""Page allocator of one cache group: pure bookkeeping, no device memory.

Like the reference's block pool (src/kipp_kv_pool.c:202-213, 258-269): all
pages start free in id order, allocation takes the head of the free list, a
freed page goes to the tail, so freed pages come back after the pages that were
never used.  Prefix sharing (the reference's content index) is not built, so a
page has one owner at most.
"""
from __future__ import annotations

from collections import deque


class OutOfPages(RuntimeError):
    """No free page is left in a group's pool."""


class PagePool:
    def __init__(self, n_pages: int):
        if n_pages <= 0:
            raise ValueError("a page pool needs at least one page")
        self.n_pages = n_pages
        self._free: deque[int] = deque(range(n_pages))
        self._owner: list[object] = [None] * n_pages

    @property
    def free_pages(self) -> int:
        return len(self._free)

    @property
    def used_pages(self) -> int:
        return self.n_pages - len(self._free)

    def owner(self, page: int):
        return self._owner[page]

    def alloc(self, owner) -> int:
        if owner is None:
            raise ValueError("a page needs an owner")
        if not self._free:
            raise OutOfPages("page pool exhausted")
        page = self._free.popleft()
        assert self._owner[page] is None, "free list held an owned page"
        self._owner[page] = owner
        return page

    def free(self, page: int, owner) -> None:
        if not 0 <= page < self.n_pages:
            raise ValueError(f"page {page} is outside the pool")
        if self._owner[page] is None:
            raise RuntimeError(f"page {page} freed twice")
        if self._owner[page] != owner:
            raise RuntimeError(f"page {page} belongs to {self._owner[page]!r}, not {owner!r}")
        self._owner[page] = None
        self._free.append(page)

    def check(self) -> None:
        """Invariant: every page is either free exactly once or owned."""
        free = list(self._free)
        if len(set(free)) != len(free):
            raise AssertionError("a page is on the free list twice")
        for p in range(self.n_pages):
            if (self._owner[p] is None) != (p in set(free)):
                raise AssertionError(f"page {p} is lost or both free and owned")
