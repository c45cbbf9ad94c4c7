from .manager import CacheGroup, CacheLayout, CacheManager, FixedState, PagedKV, RequestCache
from .pages import BlockTable, CacheAccountingError, OutOfPages, PagePool, StateSlots
from .prefix import PrefixIndex

__all__ = [
    "CacheGroup", "CacheLayout", "CacheManager", "FixedState", "PagedKV", "RequestCache", "BlockTable",
    "CacheAccountingError", "OutOfPages", "PagePool", "StateSlots", "PrefixIndex",
]
