from .manager import CacheAllocation, CacheLayout, CacheManager, LayerCache, PageGroup, RequestCache, StateArray
from .pages import PageAllocator

__all__ = [
    "CacheAllocation", "CacheLayout", "CacheManager", "LayerCache", "PageAllocator", "PageGroup",
    "RequestCache", "StateArray",
]
