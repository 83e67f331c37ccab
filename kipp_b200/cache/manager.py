"""The cache manager: pages of keys and values per group of layer runs, a
block table per request and group, and state slots.

A *group* holds the runs whose mixers declared the same ``PagedKVSpec`` (same
heads, head size and window).  Each group has its own pool of pages, its own
block tables and its own retention rule:

* full attention keeps every page until the request ends;
* a window of w gives a page back as soon as every position in it is behind
  the window of the request's next token (position < length - w + 1).

One page id addresses the same positions in every run of the group, as one
block id does in every layer of the reference's slabs (src/kipp.c:2727-2735).
Growth is all-or-nothing: if any page of a step cannot be had, the pages this
call took are returned and ``OutOfPages`` is raised with every request
unchanged (as pooled_map_blocks, src/kipp.c:3616-3635, and the batch rollback,
src/kipp.c:4043-4072).

This module is host bookkeeping only; device tensors are attached by the
engine (``CacheGroup.k`` / ``.v``).  The pools, the slots and the tables are kept
by the C++ library csrc/host/cache_core.cpp; this class groups the runs, maps
request ids to the library's integers and its error codes to exceptions.
"""
from __future__ import annotations

import ctypes
from typing import Iterable, Optional

import numpy as np

from ..parts.base import PagedKVSpec
from . import _native as N
from .pages import OutOfPages, PagePool
from .slots import OutOfSlots, StateSlots

UNMAPPED = -1


class CacheGroup:
    def __init__(self, index: int, spec: PagedKVSpec, cache_ids: list[int], page_size: int,
                 n_pages: int):
        self.index = index
        self.spec = spec
        self.cache_ids = list(cache_ids)          # ids of the runs' caches, in storage order
        self.page_size = page_size
        self.n_pages = n_pages
        self.pool: Optional[PagePool] = None      # a view of the manager's pool of this group
        self.k = None                             # device [caches, pages, kv_heads, page_size, D]
        self.v = None

    @property
    def window(self) -> Optional[int]:
        return self.spec.window

    def pages_for(self, first_pos: int, end_pos: int) -> range:
        """Logical pages that hold positions [first_pos, end_pos)."""
        if end_pos <= first_pos:
            return range(0)
        return range(first_pos // self.page_size, (end_pos - 1) // self.page_size + 1)

    def first_needed_position(self, length: int) -> int:
        """Lowest position a query at position >= ``length`` may read."""
        if self.window is None:
            return 0
        return max(0, length - self.window + 1)

    def peak_pages(self, total_tokens: int, max_step_tokens: int) -> int:
        """Most pages a request of ``total_tokens`` holds at any time when no
        step brings more than ``max_step_tokens`` of it."""
        full = -(-total_tokens // self.page_size)
        if self.window is None:
            return full
        span = self.window - 1 + max_step_tokens
        return min(full, -(-span // self.page_size) + 1)

    def bytes_per_page(self, element_size: int) -> int:
        return (2 * len(self.cache_ids) * self.spec.kv_heads * self.page_size
                * self.spec.head_dim * element_size)


class CacheManager:
    def __init__(self, specs_by_cache_id: dict[int, PagedKVSpec], page_size: int,
                 pages_per_group: int | dict[PagedKVSpec, int], max_requests: int):
        if page_size <= 0:
            raise ValueError("page_size must be positive")
        self.page_size = page_size
        by_spec: dict[PagedKVSpec, list[int]] = {}
        for cid in sorted(specs_by_cache_id):
            by_spec.setdefault(specs_by_cache_id[cid], []).append(cid)
        self.groups: list[CacheGroup] = []
        self.group_of_cache: dict[int, tuple[int, int]] = {}     # cache id -> (group, index in group)
        for gi, (spec, cids) in enumerate(by_spec.items()):
            n = pages_per_group[spec] if isinstance(pages_per_group, dict) else pages_per_group
            if n <= 0:
                raise ValueError("a page pool needs at least one page")
            self.groups.append(CacheGroup(gi, spec, cids, page_size, n))
            for j, cid in enumerate(cids):
                self.group_of_cache[cid] = (gi, j)
        if max_requests <= 0:
            raise ValueError("max_requests must be positive")
        # the pools, the slots and the tables live in the C++ library; requests are
        # 64-bit integers there
        self._lib = N.lib()
        ng = len(self.groups)
        pages = (ctypes.c_int * max(ng, 1))(*[g.n_pages for g in self.groups])
        windows = (ctypes.c_int * max(ng, 1))(*[-1 if g.window is None else g.window for g in self.groups])
        self._h = self._lib.kipp_cm_create(ng, pages, windows, page_size, max_requests)
        if not self._h:
            raise ValueError("the cache manager could not be created")
        self._owners = N.OwnerIds()
        for gi, g in enumerate(self.groups):
            g.pool = PagePool(g.n_pages, _handle=self._lib.kipp_cm_pool(self._h, gi), _owners=self._owners,
                              _keep=self)
        self.slots = StateSlots(max_requests, _handle=self._lib.kipp_cm_slots(self._h), _owners=self._owners,
                                _keep=self)
        self._held = (ctypes.c_int * max(ng, 1))()

    @classmethod
    def view_of(cls, handle, groups: list, page_size: int, max_requests: int, owners: "N.OwnerIds",
                keep=None) -> "CacheManager":
        """A face of a cache manager that someone else owns (an engine's): the
        same queries and checks, nothing is created or destroyed.  ``groups`` is a
        list of ``(PagedKVSpec, number of caches, pages)``."""
        self = cls.__new__(cls)
        self.page_size = page_size
        self._lib = N.lib()
        self._h = handle
        self._owned = False
        self._keep = keep
        self._owners = owners
        self.groups = []
        self.group_of_cache = {}
        for gi, (spec, n_caches, n_pages) in enumerate(groups):
            g = CacheGroup(gi, spec, list(range(n_caches)), page_size, n_pages)
            g.pool = PagePool(n_pages, _handle=self._lib.kipp_cm_pool(handle, gi), _owners=owners, _keep=self)
            self.groups.append(g)
        self.slots = StateSlots(max_requests, _handle=self._lib.kipp_cm_slots(handle), _owners=owners, _keep=self)
        self._held = (ctypes.c_int * max(len(self.groups), 1))()
        return self

    def __del__(self):
        h = getattr(self, "_h", None)
        if h and getattr(self, "_owned", True):
            self._lib.kipp_cm_destroy(h)
        self._h = None

    def _id(self, rid) -> int:
        i = self._owners.id_of(rid)
        if not i:
            raise KeyError(rid)
        return i

    # -- requests ---------------------------------------------------------------
    def __contains__(self, rid) -> bool:
        i = self._owners.id_of(rid)
        return bool(i) and self._lib.kipp_cm_slot(self._h, i) >= 0

    def live_requests(self) -> list:
        return [r for r in self._owners.objects() if r in self]

    def admit(self, rid) -> int:
        """Give ``rid`` a slot; it holds no pages yet.  Returns the slot."""
        if rid in self._owners:
            raise ValueError(f"request {rid!r} is already live")
        slot = self._lib.kipp_cm_admit(self._h, self._owners.id_of(rid, create=True))
        if slot < 0:
            self._owners.forget(rid)
            if slot == N.ERR_OUT_OF_SLOTS:
                raise OutOfSlots(f"all {self.slots.max_requests} request slots are in use")
            raise RuntimeError(f"admit: error {slot}")
        return slot

    def slot(self, rid) -> int:
        return self._lib.kipp_cm_slot(self._h, self._id(rid))

    def length(self, rid) -> int:
        return self._lib.kipp_cm_length(self._h, self._id(rid))

    def release(self, rid) -> None:
        """The request ended: give back all its pages and its slot."""
        rc = self._lib.kipp_cm_release(self._h, self._id(rid))
        self._owners.forget(rid)
        if rc:
            raise RuntimeError(f"release of {rid!r}: error {rc}")

    # -- growth -------------------------------------------------------------------
    def missing_pages(self, rid, new_length: int) -> list[int]:
        """Pages per group that ``reserve`` would have to take for ``rid`` to
        hold positions up to ``new_length``."""
        self._lib.kipp_cm_missing_pages(self._h, self._id(rid), new_length, self._held)
        return list(self._held[:len(self.groups)])

    def reserve(self, wants: Iterable[tuple[object, int]]) -> None:
        """Map pages so that each ``(rid, new_length)`` can be written.  Either
        every request of the call gets its pages or none does."""
        wants = list(wants)
        n = len(wants)
        if n == 0:
            return
        rids = (ctypes.c_longlong * n)(*[self._id(r) for r, _ in wants])
        lengths = (ctypes.c_int * n)(*[int(length) for _, length in wants])
        rc = self._lib.kipp_cm_reserve(self._h, n, rids, lengths)
        if rc == N.ERR_OUT_OF_PAGES:
            raise OutOfPages("page pool exhausted")
        if rc == N.ERR_ARGUMENT:
            raise ValueError("a request cannot shrink")
        if rc == N.ERR_BEHIND_WINDOW:
            raise RuntimeError("a page behind the window was asked for")
        if rc:
            raise RuntimeError(f"reserve: error {rc}")

    def advance(self, rid, new_length: int) -> None:
        """The step wrote positions up to ``new_length``.  Window groups give
        back the pages no later token can see."""
        rc = self._lib.kipp_cm_advance(self._h, self._id(rid), new_length)
        if rc == N.ERR_ARGUMENT:
            raise ValueError("a request cannot shrink")
        if rc:
            raise RuntimeError(f"advance: error {rc}")

    def truncate(self, rid, new_length: int) -> None:
        """Forget the positions from ``new_length`` on: pages that hold none of the
        remaining positions go back to their pools (the reference's session
        truncate gives back the blocks past ceil(length / block),
        src/kipp.c:3755-3768; its reset is a truncate to 0).  A window group can
        only be cut back to where the pages it still holds cover what the next
        token may see; else the call is refused and nothing changes."""
        group = ctypes.c_int(-1)
        rc = self._lib.kipp_cm_truncate(self._h, self._id(rid), new_length, ctypes.byref(group))
        if rc == N.ERR_ARGUMENT:
            raise ValueError(f"truncate to {new_length} is outside 0..{self.length(rid)}")
        if rc == N.ERR_WINDOW_REFUSES:
            raise ValueError(f"request {rid!r} cannot be cut back to {new_length}: the window of cache "
                             f"group {group.value} has already given back pages it would need")
        if rc:
            raise RuntimeError(f"truncate: error {rc}")

    # -- views ----------------------------------------------------------------------
    def table(self, rid, group: int) -> list[int]:
        i = self._id(rid)
        n = self._lib.kipp_cm_table_len(self._h, i, group)
        buf = (ctypes.c_int * max(n, 1))()
        self._lib.kipp_cm_table(self._h, i, group, buf, n)
        return list(buf[:n])

    def table_len(self, rid, group: int) -> int:
        return self._lib.kipp_cm_table_len(self._h, self._id(rid), group)

    def block_table_rows(self, rids: list, group: int, width: Optional[int] = None) -> np.ndarray:
        """int32 [len(rids), width] of physical pages, UNMAPPED where none."""
        n = len(rids)
        ids = (ctypes.c_longlong * max(n, 1))(*[self._id(r) for r in rids])
        if width is None:
            width = max([self._lib.kipp_cm_table_len(self._h, i, group) for i in ids[:n]] + [1])
        out = np.empty((n, width), dtype=np.int32)
        if n and self._lib.kipp_cm_rows(self._h, group, n, ids, width, out.ctypes.data):
            raise ValueError("block_table_rows: a table is longer than the width asked for")
        return out

    def pages_held(self, rid) -> list[int]:
        self._lib.kipp_cm_pages_held(self._h, self._id(rid), self._held)
        return list(self._held[:len(self.groups)])

    def free_pages(self) -> list[int]:
        return [g.pool.free_pages for g in self.groups]

    def check(self) -> None:
        """No page lost, held twice or free and held; tables, pools and slots agree."""
        if self._lib.kipp_cm_check(self._h):
            raise AssertionError("the cache manager's tables, pools and slots disagree "
                                 "(a page lost, held twice, or both free and held)")
