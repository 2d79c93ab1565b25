from .allocators import CacheCapacityError, IndexAllocator
from .needs import KVNeed, StateNeed
from .sequence_cache import PAGE_SIZE, CacheView, KVGroup, SequenceCache, StateGroup, pages_for

__all__ = ["CacheCapacityError", "IndexAllocator", "KVNeed", "StateNeed", "PAGE_SIZE", "CacheView",
           "KVGroup", "SequenceCache", "StateGroup", "pages_for"]
