"""The cache's bookkeeping, as Python sees it: a view of the host's ``PagedKVCache`` (``csrc/host/cache.cpp``).

A slot per live sequence holds its length and, per cache group, the pages it owns; a cache group is the set of
schedule entries whose mixers asked for the same (KV heads, head size, window) and has storage of its own; a
windowed group gives pages back as they leave the window; page 0 is never handed out.  An engine holds such a
cache with device pools; this class creates the bookkeeping alone (no device memory), which is what the host-side
tests drive.  Reference: per-layer arrays ``[capacity][kv_dim]`` for one sequence (fastgguf.c:4114-4115,
:4449-4450), rings for sliding-window layers (:4427-4436), borrowed caches (:4745-4751).
"""
from __future__ import annotations

import json
from ctypes import byref, c_int, c_void_p
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np

from .. import capi
from ..capi import CacheError, CacheFull

__all__ = ["CacheError", "CacheFull", "CacheRequest", "PagedKVCache", "cache_bytes"]


@dataclass(frozen=True)
class CacheRequest:
    """Keys and values a mixer keeps per position.  ``window`` None keeps every position; an integer keeps the
    last ``window`` positions.  Requests that agree in all fields share a cache group."""

    n_kv_heads: int
    head_dim: int
    window: Optional[int] = None


def _requests_json(requests: Dict[int, CacheRequest]) -> bytes:
    return json.dumps([{"entry": int(e), "n_kv_heads": r.n_kv_heads, "head_dim": r.head_dim, "window": r.window}
                       for e, r in sorted(requests.items())]).encode("utf-8")


def cache_bytes(requests: Dict[int, CacheRequest], max_tokens: int, page_size: int = 64, dtype="bfloat16") -> dict:
    """{"bytes_per_token", "pages", "bytes"} of the pools such a cache would take; nothing is allocated."""
    from ..weights import dtype_code
    return capi.take_json(capi.lib().fg_cache_bytes, _requests_json(requests), int(max_tokens), page_size, dtype_code(dtype))


class PagedKVCache:
    def __init__(self, requests: Dict[int, CacheRequest], *, max_tokens: int, max_seq_len: int, n_slots: int,
                 page_size: int = 64):
        out = c_void_p()
        capi.check(capi.lib().fg_cache_create(_requests_json(requests), int(max_tokens), int(max_seq_len), int(n_slots),
                                              int(page_size), byref(out)))
        self._handle = out
        self.page_size, self.n_slots, self.max_seq_len = page_size, n_slots, max_seq_len

    def __del__(self):
        h, self._handle = getattr(self, "_handle", None), None
        if h:
            try:
                capi.lib().fg_cache_destroy(h)
            except Exception:
                pass

    def _int(self, fn, *args) -> int:
        out = c_int()
        capi.check(fn(self._handle, *args, byref(out)))
        return out.value

    def info(self) -> dict:
        return capi.take_json(capi.lib().fg_cache_info, self._handle)

    @property
    def groups(self) -> List[dict]:
        return self.info()["groups"]

    @property
    def group_of_entry(self) -> Dict[int, int]:
        return {e: gi for gi, g in enumerate(self.groups) for e in g["entries"]}

    def acquire(self) -> int:
        return self._int(capi.lib().fg_cache_acquire)

    def release(self, slot: int) -> None:
        capi.check(capi.lib().fg_cache_release(self._handle, int(slot)))

    def length(self, slot: int) -> int:
        return self._int(capi.lib().fg_cache_length, int(slot))

    def live_slots(self) -> List[int]:
        return list(self.info()["live_slots"])

    @staticmethod
    def _steps(steps: Sequence[Tuple[int, int]]):
        slots, n = capi.int_array([s for s, _ in steps])
        news, _ = capi.int_array([k for _, k in steps])
        return n, slots, news

    def reserve(self, steps: Sequence[Tuple[int, int]]) -> None:
        """Make room for ``n_new`` more tokens in each ``(slot, n_new)``; all or nothing."""
        capi.check(capi.lib().fg_cache_reserve(self._handle, *self._steps(steps)))

    def commit(self, steps: Sequence[Tuple[int, int]]) -> None:
        """The step ran: lengths grow, and windowed groups give back pages that left the window."""
        capi.check(capi.lib().fg_cache_commit(self._handle, *self._steps(steps)))

    def pages_needed(self, slot: int, n_new: int) -> List[int]:
        out = (c_int * max(1, len(self.groups)))()
        capi.check(capi.lib().fg_cache_pages_needed(self._handle, int(slot), int(n_new), out))
        return list(out)[:len(self.groups)]

    def free_pages(self, gi: int = 0) -> int:
        return self._int(capi.lib().fg_cache_free_pages, int(gi))

    def block_table(self, gi: int, slots: Sequence[int], width: int) -> np.ndarray:
        table = np.zeros((len(slots), width), dtype=np.int32)
        row = (c_int * max(1, width))()
        for i, s in enumerate(slots):
            capi.check(capi.lib().fg_cache_block_table(self._handle, int(gi), int(s), int(width), row))
            table[i] = np.frombuffer(row, dtype=np.int32, count=width)
        return table

    def check(self) -> None:
        """Raise if a page or slot is lost, held twice or freed twice."""
        capi.check(capi.lib().fg_cache_check(self._handle))
