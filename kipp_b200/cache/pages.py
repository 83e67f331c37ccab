"""Page allocator of one cache group: pure bookkeeping, no device memory.

Like the reference's block pool (src/kipp_kv_pool.c:202-213, 258-269): all
pages start free in id order, allocation takes the head of the free list, a
freed page goes to the tail, so freed pages come back after the pages that were
never used.  Prefix sharing (the reference's content index) is not built, so a
page has one owner at most.  The list and the owners live in the C++ library
(csrc/host/cache_core.cpp); this class maps owners to its integers and its
error codes to exceptions.
"""
from __future__ import annotations

from . import _native as N


class OutOfPages(RuntimeError):
    """No free page is left in a group's pool."""


class PagePool:
    def __init__(self, n_pages: int, *, _handle=None, _owners: "N.OwnerIds | None" = None, _keep=None):
        if n_pages <= 0:
            raise ValueError("a page pool needs at least one page")
        self.n_pages = n_pages
        self._lib = N.lib()
        self._own_handle = _handle is None
        self._h = self._lib.kipp_pool_create(n_pages) if _handle is None else _handle
        self._owners = _owners if _owners is not None else N.OwnerIds()
        self._held: dict = {}                 # stand-alone use: pages per owner, to forget owners without pages
        self._keep = _keep                    # the manager whose pool this is a view of

    def __del__(self):
        if getattr(self, "_own_handle", False) and self._h:
            self._lib.kipp_pool_destroy(self._h)
            self._h = None

    @property
    def free_pages(self) -> int:
        return self._lib.kipp_pool_free_pages(self._h)

    @property
    def used_pages(self) -> int:
        return self.n_pages - self.free_pages

    def owner(self, page: int):
        i = self._lib.kipp_pool_owner(self._h, page)
        return None if i == N.NO_OWNER else self._owners.obj_of(i)

    def alloc(self, owner) -> int:
        if owner is None:
            raise ValueError("a page needs an owner")
        page = self._lib.kipp_pool_alloc(self._h, self._owners.id_of(owner, create=True))
        if page == N.ERR_OUT_OF_PAGES:
            if self._own_handle and not self._held.get(owner):
                self._owners.forget(owner)
            raise OutOfPages("page pool exhausted")
        if self._own_handle:
            self._held[owner] = self._held.get(owner, 0) + 1
        return page

    def free(self, page: int, owner) -> None:
        if not 0 <= page < self.n_pages:
            raise ValueError(f"page {page} is outside the pool")
        rc = self._lib.kipp_pool_free(self._h, page, self._owners.id_of(owner))
        if rc == N.ERR_FREED_TWICE:
            raise RuntimeError(f"page {page} freed twice")
        if rc == N.ERR_NOT_OWNER:
            raise RuntimeError(f"page {page} belongs to {self.owner(page)!r}, not {owner!r}")
        if rc:
            raise RuntimeError(f"page {page}: error {rc}")
        if self._own_handle:
            left = self._held.get(owner, 1) - 1
            if left:
                self._held[owner] = left
            else:
                self._held.pop(owner, None)
                self._owners.forget(owner)

    def check(self) -> None:
        """Invariant: every page is either free exactly once or owned."""
        if self._lib.kipp_pool_check(self._h):
            raise AssertionError("a page is lost, on the free list twice, or both free and owned")
