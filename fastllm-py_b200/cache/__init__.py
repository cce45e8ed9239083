from .manager import CacheManager, PageGroup, RequestCache
from .needs import FixedState, PagedKV, PagedNeed
from .views import PagedCacheView, StateView
from .pages import OutOfPages, PagePool, SlotPool

__all__ = ["CacheManager", "PageGroup", "RequestCache", "FixedState", "PagedKV", "PagedNeed",
           "PagedCacheView", "StateView", "OutOfPages", "PagePool", "SlotPool"]
