from .manager import CacheError, CacheManager, OutOfPages, PagePool, SeqCache
from .spec import CacheLayout, CacheSpec, KVSpec, PlaneRef, StateSpec

__all__ = ["CacheError", "CacheManager", "OutOfPages", "PagePool", "SeqCache",
           "CacheLayout", "CacheSpec", "KVSpec", "PlaneRef", "StateSpec"]
