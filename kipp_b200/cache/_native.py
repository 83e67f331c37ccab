"""ctypes bindings of the cache manager's C functions (csrc/host/cache_core.cpp,
part of the host core's library)."""
from __future__ import annotations

import ctypes

OK = 0
ERR_OUT_OF_PAGES = -1
ERR_OUT_OF_SLOTS = -2
ERR_ARGUMENT = -3
ERR_BEHIND_WINDOW = -4
ERR_CHECK = -5
ERR_FREED_TWICE = -6
ERR_NOT_OWNER = -7
ERR_WINDOW_REFUSES = -8
NO_OWNER = -(1 << 63)

_vp, _i, _ll = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
_ip, _llp = ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_longlong)

_SIGNATURES = {
    "kipp_pool_create": (_vp, [_i]), "kipp_pool_destroy": (None, [_vp]),
    "kipp_pool_alloc": (_i, [_vp, _ll]), "kipp_pool_free": (_i, [_vp, _i, _ll]),
    "kipp_pool_free_pages": (_i, [_vp]), "kipp_pool_owner": (_ll, [_vp, _i]), "kipp_pool_check": (_i, [_vp]),
    "kipp_slots_create": (_vp, [_i]), "kipp_slots_destroy": (None, [_vp]),
    "kipp_slots_alloc": (_i, [_vp, _ll]), "kipp_slots_free": (_i, [_vp, _i, _ll]),
    "kipp_slots_free_count": (_i, [_vp]), "kipp_slots_check": (_i, [_vp]),
    "kipp_cm_create": (_vp, [_i, _ip, _ip, _i, _i]), "kipp_cm_destroy": (None, [_vp]),
    "kipp_cm_pool": (_vp, [_vp, _i]), "kipp_cm_slots": (_vp, [_vp]),
    "kipp_cm_admit": (_i, [_vp, _ll]), "kipp_cm_release": (_i, [_vp, _ll]),
    "kipp_cm_slot": (_i, [_vp, _ll]), "kipp_cm_length": (_i, [_vp, _ll]),
    "kipp_cm_missing_pages": (_i, [_vp, _ll, _i, _ip]),
    "kipp_cm_reserve": (_i, [_vp, _i, _llp, _ip]),
    "kipp_cm_advance": (_i, [_vp, _ll, _i]), "kipp_cm_truncate": (_i, [_vp, _ll, _i, _ip]),
    "kipp_cm_table_len": (_i, [_vp, _ll, _i]), "kipp_cm_table": (_i, [_vp, _ll, _i, _ip, _i]),
    "kipp_cm_rows": (_i, [_vp, _i, _i, _llp, _i, _vp]),
    "kipp_cm_pages_held": (_i, [_vp, _ll, _ip]), "kipp_cm_check": (_i, [_vp]),
}
_lib = None


def lib() -> ctypes.CDLL:
    """The library, built at first use (there is no Python stand-in)."""
    global _lib
    if _lib is None:
        from ..csrc import build
        loaded = build.load_host_library()
        for name, (res, args) in _SIGNATURES.items():
            fn = getattr(loaded, name)
            fn.restype, fn.argtypes = res, args
        _lib = loaded
    return _lib


class OwnerIds:
    """Owners are any hashable objects here and 64-bit integers in the library."""

    def __init__(self):
        self._ids: dict = {}
        self._objs: dict = {}
        self._next = 1

    def id_of(self, obj, create: bool = False) -> int:
        i = self._ids.get(obj)
        if i is None:
            if not create:
                return 0                     # no owner has this id
            i = self._next
            self._next += 1
            self._ids[obj] = i
            self._objs[i] = obj
        return i

    def obj_of(self, i: int):
        return self._objs.get(i)

    def forget(self, obj) -> None:
        i = self._ids.pop(obj, None)
        if i is not None:
            del self._objs[i]

    def __contains__(self, obj) -> bool:
        return obj in self._ids

    def objects(self) -> list:
        return list(self._ids)
