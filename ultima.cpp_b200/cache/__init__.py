"""The cache: slots, pages of keys and values for each group of layers, fixed-size state."""
from .book import CacheError, PageAllocator, SlotBook
from .store import Cache, KVGroup, StateGroup, KVView, RunCache, PAGE

__all__ = ["CacheError", "PageAllocator", "SlotBook", "Cache", "KVGroup", "StateGroup", "KVView",
           "RunCache", "PAGE"]
