"""Cache manager: paged keys/values in groups, block tables, fixed-size state slots."""
from .manager import CacheGroup, CacheManager, KVNeed, RequestCache, StateNeed
from .pages import OutOfPages, PagePool, SlotPool

__all__ = ["CacheGroup", "CacheManager", "KVNeed", "RequestCache", "StateNeed",
           "OutOfPages", "PagePool", "SlotPool"]
