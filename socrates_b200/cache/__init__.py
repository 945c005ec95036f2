from .allocator import OutOfPages, PageAllocator, pages_for
from .manager import CacheManager, CacheNeeds, PagedKVSpec, PageGroup, StateSpec

__all__ = ["OutOfPages", "PageAllocator", "pages_for", "CacheManager", "CacheNeeds",
           "PagedKVSpec", "PageGroup", "StateSpec"]
