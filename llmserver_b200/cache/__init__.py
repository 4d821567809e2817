from .pool import KVCacheExhaustedError, KVCacheStateError, PagePool
from .manager import CacheGroup, CacheManager, KVPagesNeed, StateNeed, StateSlots, RELEASED

__all__ = ["KVCacheExhaustedError", "KVCacheStateError", "PagePool", "CacheGroup", "CacheManager", "KVPagesNeed",
           "StateNeed", "StateSlots", "RELEASED"]
