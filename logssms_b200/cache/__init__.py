from .manager import CacheManager, CacheNeeds, KVNeed, PagedNeed, PagedTensor, PageGroup, RequestCache, StateNeed
from .pools import FreeList, OutOfPages

__all__ = ["CacheManager", "CacheNeeds", "KVNeed", "PagedNeed", "PagedTensor", "PageGroup", "RequestCache", "StateNeed", "FreeList", "OutOfPages"]
