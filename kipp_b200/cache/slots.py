"""Slots for per-request state of fixed size.

Every live request holds one slot index.  A mixer that declares a
``StateSpec`` gets a device tensor ``[max_requests, *shape]`` per run, indexed
by slot and zeroed when the slot is handed out.  The Qwen3 decoder has no such
state; the slot still numbers the request's row in the block tables.  (The
reference keeps the fixed-size per-request data in host structs,
src/kipp.c:154-164 and src/kipp_server.c:869-887.)
"""
from __future__ import annotations


class OutOfSlots(RuntimeError):
    pass


class StateSlots:
    def __init__(self, max_requests: int):
        if max_requests <= 0:
            raise ValueError("max_requests must be positive")
        self.max_requests = max_requests
        self._free = list(range(max_requests - 1, -1, -1))
        self._owner: dict[int, object] = {}

    @property
    def free_slots(self) -> int:
        return len(self._free)

    def alloc(self, owner) -> int:
        if not self._free:
            raise OutOfSlots(f"all {self.max_requests} request slots are in use")
        slot = self._free.pop()
        self._owner[slot] = owner
        return slot

    def free(self, slot: int, owner) -> None:
        if self._owner.get(slot) != owner or slot not in self._owner:
            raise RuntimeError(f"slot {slot} is not held by {owner!r}")
        del self._owner[slot]
        self._free.append(slot)

    def check(self) -> None:
        held = set(self._owner)
        free = set(self._free)
        if len(free) != len(self._free) or held & free or len(held | free) != self.max_requests:
            raise AssertionError("a slot is lost or held twice")
