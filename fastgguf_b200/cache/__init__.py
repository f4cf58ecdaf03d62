"""Paged key/value cache with per-sequence slots (bookkeeping view of the host's cache)."""
from .paged import CacheError, CacheFull, CacheRequest, PagedKVCache, cache_bytes

__all__ = ["CacheError", "CacheFull", "CacheRequest", "PagedKVCache", "cache_bytes"]
