from .pools import IdPool, PoolError
from .manager import CacheManager, OutOfPages, OutOfSlots, PagedKVView, RequestCache, SlotView

__all__ = ["IdPool", "PoolError", "CacheManager", "OutOfPages", "OutOfSlots", "PagedKVView", "RequestCache",
           "SlotView"]
