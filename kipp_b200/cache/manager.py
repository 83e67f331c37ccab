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
engine (``CacheGroup.k`` / ``.v``).
"""
from __future__ import annotations

import dataclasses
from typing import Iterable, Optional

import numpy as np

from ..parts.base import PagedKVSpec
from .pages import OutOfPages, PagePool
from .slots import StateSlots

UNMAPPED = -1


@dataclasses.dataclass
class _RequestCache:
    slot: int
    length: int = 0
    # per group: logical page index -> physical page (UNMAPPED if none)
    tables: list = dataclasses.field(default_factory=list)
    # per group: first logical page that may still be mapped (pages before it
    # were given back by the window)
    first_live: list = dataclasses.field(default_factory=list)
    # per group: int32 mirror of ``tables`` (grown by doubling) so that block
    # tables of a step are copied, not converted from lists
    mirrors: list = dataclasses.field(default_factory=list)

    def set_page(self, group: int, logical: int, page: int) -> None:
        table = self.tables[group]
        while len(table) <= logical:
            table.append(UNMAPPED)
        table[logical] = page
        mirror = self.mirrors[group]
        if logical >= mirror.shape[0]:
            grown = np.full(max(2 * mirror.shape[0], logical + 1, 16), UNMAPPED, dtype=np.int32)
            grown[:mirror.shape[0]] = mirror
            self.mirrors[group] = mirror = grown
        mirror[logical] = page

    def trim(self, group: int) -> None:
        """Drop trailing unmapped entries (after a roll-back)."""
        table = self.tables[group]
        while table and table[-1] == UNMAPPED:
            table.pop()


class CacheGroup:
    def __init__(self, index: int, spec: PagedKVSpec, cache_ids: list[int], page_size: int,
                 n_pages: int):
        self.index = index
        self.spec = spec
        self.cache_ids = list(cache_ids)          # ids of the runs' caches, in storage order
        self.page_size = page_size
        self.pool = PagePool(n_pages)
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
        self.slots = StateSlots(max_requests)
        by_spec: dict[PagedKVSpec, list[int]] = {}
        for cid in sorted(specs_by_cache_id):
            by_spec.setdefault(specs_by_cache_id[cid], []).append(cid)
        self.groups: list[CacheGroup] = []
        self.group_of_cache: dict[int, tuple[int, int]] = {}     # cache id -> (group, index in group)
        for gi, (spec, cids) in enumerate(by_spec.items()):
            n = pages_per_group[spec] if isinstance(pages_per_group, dict) else pages_per_group
            self.groups.append(CacheGroup(gi, spec, cids, page_size, n))
            for j, cid in enumerate(cids):
                self.group_of_cache[cid] = (gi, j)
        self._requests: dict[object, _RequestCache] = {}

    # -- requests ---------------------------------------------------------------
    def __contains__(self, rid) -> bool:
        return rid in self._requests

    def live_requests(self) -> list:
        return list(self._requests)

    def admit(self, rid) -> int:
        """Give ``rid`` a slot; it holds no pages yet.  Returns the slot."""
        if rid in self._requests:
            raise ValueError(f"request {rid!r} is already live")
        slot = self.slots.alloc(rid)
        self._requests[rid] = _RequestCache(slot=slot, tables=[[] for _ in self.groups],
                                            first_live=[0 for _ in self.groups],
                                            mirrors=[np.full(16, UNMAPPED, dtype=np.int32)
                                                     for _ in self.groups])
        return slot

    def slot(self, rid) -> int:
        return self._requests[rid].slot

    def length(self, rid) -> int:
        return self._requests[rid].length

    def release(self, rid) -> None:
        """The request ended: give back all its pages and its slot."""
        rc = self._requests.pop(rid)
        for g, table in zip(self.groups, rc.tables):
            for page in table:
                if page != UNMAPPED:
                    g.pool.free(page, rid)
        self.slots.free(rc.slot, rid)

    # -- growth -------------------------------------------------------------------
    def missing_pages(self, rid, new_length: int) -> list[int]:
        """Pages per group that ``reserve`` would have to take for ``rid`` to
        hold positions up to ``new_length``."""
        rc = self._requests[rid]
        out = []
        for gi, g in enumerate(self.groups):
            table = rc.tables[gi]
            out.append(sum(1 for lp in g.pages_for(rc.length, new_length)
                           if lp >= len(table) or table[lp] == UNMAPPED))
        return out

    def reserve(self, wants: Iterable[tuple[object, int]]) -> None:
        """Map pages so that each ``(rid, new_length)`` can be written.  Either
        every request of the call gets its pages or none does."""
        taken: list[tuple[int, object, int, int]] = []       # (group, rid, logical, page)
        try:
            for rid, new_length in wants:
                rc = self._requests[rid]
                if new_length < rc.length:
                    raise ValueError("a request cannot shrink")
                for gi, g in enumerate(self.groups):
                    table = rc.tables[gi]
                    for lp in g.pages_for(rc.length, new_length):
                        if lp >= len(table) or table[lp] == UNMAPPED:
                            if lp < rc.first_live[gi]:
                                raise RuntimeError("a page behind the window was asked for")
                            page = g.pool.alloc(rid)
                            rc.set_page(gi, lp, page)
                            taken.append((gi, rid, lp, page))
        except OutOfPages:
            for gi, rid, lp, page in reversed(taken):
                self.groups[gi].pool.free(page, rid)
                self._requests[rid].set_page(gi, lp, UNMAPPED)
            for rid, _ in wants:
                rc = self._requests.get(rid)
                if rc is None:
                    continue
                for gi in range(len(self.groups)):  # drop trailing holes the call made
                    rc.trim(gi)
            raise

    def advance(self, rid, new_length: int) -> None:
        """The step wrote positions up to ``new_length``.  Window groups give
        back the pages no later token can see."""
        rc = self._requests[rid]
        if new_length < rc.length:
            raise ValueError("a request cannot shrink")
        rc.length = new_length
        for gi, g in enumerate(self.groups):
            if g.window is None:
                continue
            table = rc.tables[gi]
            keep_from = g.first_needed_position(new_length) // g.page_size
            for lp in range(rc.first_live[gi], min(keep_from, len(table))):
                if table[lp] != UNMAPPED:
                    g.pool.free(table[lp], rid)
                    rc.set_page(gi, lp, UNMAPPED)
            rc.first_live[gi] = max(rc.first_live[gi], min(keep_from, len(table)))

    def truncate(self, rid, new_length: int) -> None:
        """Forget the positions from ``new_length`` on: pages that hold none of the
        remaining positions go back to their pools (the reference's session
        truncate gives back the blocks past ceil(length / block),
        src/kipp.c:3755-3768; its reset is a truncate to 0).  A window group can
        only be cut back to where the pages it still holds cover what the next
        token may see; else the call is refused and nothing changes."""
        rc = self._requests[rid]
        if new_length < 0 or new_length > rc.length:
            raise ValueError(f"truncate to {new_length} is outside 0..{rc.length}")
        for gi, g in enumerate(self.groups):
            if g.window is None or new_length == 0:
                continue
            first_page = g.first_needed_position(new_length) // g.page_size
            if first_page < rc.first_live[gi]:
                raise ValueError(f"request {rid!r} cannot be cut back to {new_length}: the window of cache "
                                 f"group {gi} has already given back pages it would need")
        for gi, g in enumerate(self.groups):
            table = rc.tables[gi]
            keep = -(-new_length // g.page_size)              # pages with positions below new_length
            for lp in range(keep, len(table)):
                if table[lp] != UNMAPPED:
                    g.pool.free(table[lp], rid)
                    rc.set_page(gi, lp, UNMAPPED)
            del table[keep:]
            if new_length == 0:
                rc.first_live[gi] = 0
            else:
                rc.first_live[gi] = min(rc.first_live[gi], keep)
        rc.length = new_length

    # -- views ----------------------------------------------------------------------
    def table(self, rid, group: int) -> list[int]:
        return self._requests[rid].tables[group]

    def block_table_rows(self, rids: list, group: int, width: Optional[int] = None) -> np.ndarray:
        """int32 [len(rids), width] of physical pages, UNMAPPED where none."""
        reqs = [self._requests[r] for r in rids]
        lens = [len(rc.tables[group]) for rc in reqs]
        if width is None:
            width = max(lens + [1])
        out = np.full((len(rids), width), UNMAPPED, dtype=np.int32)
        for i, (rc, n) in enumerate(zip(reqs, lens)):
            if n:
                out[i, :n] = rc.mirrors[group][:n]
        return out

    def pages_held(self, rid) -> list[int]:
        return [sum(1 for p in t if p != UNMAPPED) for t in self._requests[rid].tables]

    def free_pages(self) -> list[int]:
        return [g.pool.free_pages for g in self.groups]

    def check(self) -> None:
        """No page lost, held twice or free and held; tables and pools agree."""
        for gi, g in enumerate(self.groups):
            g.pool.check()
            seen: dict[int, object] = {}
            for rid, rc in self._requests.items():
                for page in rc.tables[gi]:
                    if page == UNMAPPED:
                        continue
                    if page in seen:
                        raise AssertionError(f"page {page} of group {gi} is held twice")
                    seen[page] = rid
                    if g.pool.owner(page) != rid:
                        raise AssertionError(f"page {page} of group {gi}: table and pool disagree")
            for rid, rc in self._requests.items():
                n = len(rc.tables[gi])
                if rc.mirrors[gi][:n].tolist() != rc.tables[gi]:
                    raise AssertionError(f"group {gi}: the int32 mirror of {rid!r}'s table is stale")
            if len(seen) != g.pool.used_pages:
                raise AssertionError(f"group {gi}: {g.pool.used_pages - len(seen)} pages are lost")
        self.slots.check()
