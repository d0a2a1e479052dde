from .manager import CacheError, CacheGroupSpec, CacheManager, PagePool, SlotPool, group_runs
from .storage import CacheStorage, page_bytes

__all__ = ["CacheError", "CacheGroupSpec", "CacheManager", "CacheStorage", "PagePool", "SlotPool",
           "group_runs", "page_bytes"]
