from .cache import PAGE_SIZE, Cache, CacheEntry, CacheSpec, KVGroup, KVSpec, StateGroup, StateSpec
from .pages import CacheError, CacheFull, PagePool, SlotTable

__all__ = ["PAGE_SIZE", "Cache", "CacheEntry", "CacheSpec", "KVGroup", "KVSpec", "StateGroup", "StateSpec",
           "CacheError", "CacheFull", "PagePool", "SlotTable"]
