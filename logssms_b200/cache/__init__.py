from .manager import CacheManager, CacheNeeds, KVNeed, PageGroup, RequestCache, StateNeed
from .pools import FreeList, OutOfPages

__all__ = ["CacheManager", "CacheNeeds", "KVNeed", "PageGroup", "RequestCache", "StateNeed", "FreeList", "OutOfPages"]
