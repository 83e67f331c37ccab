from .manager import UNMAPPED, CacheGroup, CacheManager
from .pages import OutOfPages, PagePool
from .slots import OutOfSlots, StateSlots

__all__ = ["UNMAPPED", "CacheGroup", "CacheManager", "OutOfPages", "PagePool", "OutOfSlots",
           "StateSlots"]
