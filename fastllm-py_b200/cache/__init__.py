from .manager import CacheManager, PageGroup, RequestCache
from .needs import FixedState, PagedKV
from .pages import OutOfPages, PagePool, SlotPool

__all__ = ["CacheManager", "PageGroup", "RequestCache", "FixedState", "PagedKV",
           "OutOfPages", "PagePool", "SlotPool"]
