from .allocator import CacheError, FreeList, PageTableHost
from .cache import PAGE_SIZE, Cache, CacheUnit, KVRequest, KVUnit, StateRequest

__all__ = ["CacheError", "FreeList", "PageTableHost", "PAGE_SIZE", "Cache", "CacheUnit", "KVRequest", "KVUnit",
           "StateRequest"]
