"""Slots for per-request state of fixed size.

Every live request holds one slot index.  A mixer that declares a
``StateSpec`` gets a device tensor ``[max_requests, *shape]`` per run, indexed
by slot and zeroed when the slot is handed out.  The Qwen3 decoder has no such
state; the slot still numbers the request's row in the block tables.  (The
reference keeps the fixed-size per-request data in host structs,
src/kipp.c:154-164 and src/kipp_server.c:869-887.)  The free stack and the
owners live in the C++ library (csrc/host/cache_core.cpp).
"""
from __future__ import annotations

from . import _native as N


class OutOfSlots(RuntimeError):
    pass


class StateSlots:
    def __init__(self, max_requests: int, *, _handle=None, _owners: "N.OwnerIds | None" = None, _keep=None):
        if max_requests <= 0:
            raise ValueError("max_requests must be positive")
        self.max_requests = max_requests
        self._lib = N.lib()
        self._own_handle = _handle is None
        self._h = self._lib.kipp_slots_create(max_requests) if _handle is None else _handle
        self._owners = _owners if _owners is not None else N.OwnerIds()
        self._keep = _keep

    def __del__(self):
        if getattr(self, "_own_handle", False) and self._h:
            self._lib.kipp_slots_destroy(self._h)
            self._h = None

    @property
    def free_slots(self) -> int:
        return self._lib.kipp_slots_free_count(self._h)

    def alloc(self, owner) -> int:
        known = owner in self._owners
        slot = self._lib.kipp_slots_alloc(self._h, self._owners.id_of(owner, create=True))
        if slot == N.ERR_OUT_OF_SLOTS:
            if self._own_handle and not known:
                self._owners.forget(owner)
            raise OutOfSlots(f"all {self.max_requests} request slots are in use")
        return slot

    def free(self, slot: int, owner) -> None:
        if self._lib.kipp_slots_free(self._h, slot, self._owners.id_of(owner)):
            raise RuntimeError(f"slot {slot} is not held by {owner!r}")
        if self._own_handle:
            self._owners.forget(owner)

    def check(self) -> None:
        if self._lib.kipp_slots_check(self._h):
            raise AssertionError("a slot is lost or held twice")
