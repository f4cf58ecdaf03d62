"""Paged key/value cache with per-sequence slots and fixed-size per-sequence state."""
from .paged import CacheError, CacheFull, CacheGroup, PagedKVCache, StatePool

__all__ = ["CacheError", "CacheFull", "CacheGroup", "PagedKVCache", "StatePool"]
