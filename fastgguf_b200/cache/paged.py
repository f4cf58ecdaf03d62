"""The cache: a slot per sequence, pages of keys and values per layer, and per-sequence state.

The reference keeps, per layer that owns a cache, two float arrays ``[capacity][kv_dim]``
written at ``pos % capacity`` (fastgguf.c:4114-4115, :4449-4450, :4720), for ONE sequence per
model; sliding-window layers get a short ring of their own while global layers get the full
context (:4427-4436), and shared-KV layers own nothing and read a donor's arrays (:4745-4751).
Per-sequence scalars (position, RNG) are scattered over locals and structs (:5243, :3974).

Here many sequences share the storage:

* a **slot** per live sequence holds its length and, per cache group, the list of pages it owns;
* a **cache group** is the set of schedule entries whose mixers asked for the same
  (KV heads, head size, window); it has storage of its own - one page pool per entry - and one
  page table per sequence, so a full-attention group and a windowed group never share pages;
* a page holds ``page_size`` consecutive positions of one sequence for all KV heads of one
  entry: pool layout ``[pages, kv_heads, page_size, head_dim]``;
* a windowed group gives pages back as soon as every position in them has left the window;
* page 0 of every group is never handed out: padded rows of a fixed-shape step write there;
* beside the pages, :class:`StatePool` keeps ``[n_slots, *shape]`` tensors for mixers that
  ask for fixed-size state; a slot's rows are zeroed when a sequence takes the slot.

All bookkeeping is on the host and checked: a page or a slot can neither be lost, held twice
nor freed twice (``check()`` proves it, tests call it after every operation).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..parts.base import CacheRequest, StateRequest


class CacheError(RuntimeError):
    pass


class CacheFull(CacheError):
    """No free slot, or not enough free pages for the tokens a step brings."""


@dataclass
class CacheGroup:
    request: CacheRequest
    entries: List[int]                         # schedule entries that own a pool in this group
    n_pages: int                               # pages in each pool, the reserved page 0 included
    free: List[int] = field(default_factory=list)
    k_pools: Dict[int, torch.Tensor] = field(default_factory=dict)
    v_pools: Dict[int, torch.Tensor] = field(default_factory=dict)


@dataclass
class _Slot:
    length: int = 0
    live: bool = False
    pages: List[Dict[int, int]] = field(default_factory=list)   # per group: page index in sequence -> page id


class PagedKVCache:
    def __init__(self, requests: Dict[int, CacheRequest], *, max_tokens: int, max_seq_len: int,
                 n_slots: int, page_size: int = 64, dtype: torch.dtype = torch.bfloat16,
                 device: Optional[torch.device] = None, allocate: bool = True):
        """``requests``: schedule entry -> what its mixer keeps.  ``max_tokens``: most tokens held
        by live sequences at any time, each sequence counted rounded up to a page."""
        if page_size <= 0 or max_tokens <= 0 or n_slots <= 0:
            raise CacheError("page_size, max_tokens and n_slots must be positive")
        self.page_size = page_size
        self.n_slots = n_slots
        self.max_seq_len = max_seq_len
        self.table_width = min(64, (max_seq_len + page_size - 1) // page_size)   # grows on demand
        self.dtype, self.device = dtype, device
        n_pages = (max_tokens + page_size - 1) // page_size + 1      # + the reserved page 0
        self.groups: List[CacheGroup] = []
        self.group_of_entry: Dict[int, int] = {}
        for entry in sorted(requests):
            req = requests[entry]
            for gi, g in enumerate(self.groups):
                if g.request == req:
                    g.entries.append(entry)
                    self.group_of_entry[entry] = gi
                    break
            else:
                self.groups.append(CacheGroup(req, [entry], n_pages))
                self.group_of_entry[entry] = len(self.groups) - 1
        for g in self.groups:
            g.free = list(range(n_pages - 1, 0, -1))                 # pop() hands out low ids first
            if allocate:
                shape = (n_pages, g.request.n_kv_heads, page_size, g.request.head_dim)
                for e in g.entries:
                    g.k_pools[e] = torch.zeros(shape, dtype=dtype, device=device)
                    g.v_pools[e] = torch.zeros(shape, dtype=dtype, device=device)
        self._slots = [_Slot(pages=[{} for _ in self.groups]) for _ in range(n_slots)]
        self._free_slots = list(range(n_slots - 1, -1, -1))
        # host mirror of the page tables: [group][slot, page index] -> page id (0 where none)
        self.tables = [np.zeros((n_slots, self.table_width), dtype=np.int32) for _ in self.groups]

    # ------------------------------------------------------------------ slots
    def acquire(self) -> int:
        if not self._free_slots:
            raise CacheFull(f"all {self.n_slots} sequence slots are in use")
        s = self._free_slots.pop()
        slot = self._slots[s]
        assert not slot.live and slot.length == 0 and all(not p for p in slot.pages)
        slot.live = True
        return s

    def release(self, s: int) -> None:
        slot = self._slot(s)
        for gi, g in enumerate(self.groups):
            for page in slot.pages[gi].values():
                g.free.append(page)
            slot.pages[gi].clear()
            self.tables[gi][s, :] = 0
        slot.length, slot.live = 0, False
        self._free_slots.append(s)

    def _slot(self, s: int) -> _Slot:
        if not (0 <= s < self.n_slots):
            raise CacheError(f"slot {s} does not exist (there are {self.n_slots})")
        slot = self._slots[s]
        if not slot.live:
            raise CacheError(f"slot {s} is not held by a sequence (released twice, or never acquired)")
        return slot

    def length(self, s: int) -> int:
        return self._slot(s).length

    def live_slots(self) -> List[int]:
        return [i for i, s in enumerate(self._slots) if s.live]

    # ------------------------------------------------------------------ pages
    def _first_needed_page(self, g: CacheGroup, new_length: int) -> int:
        """Index (within a sequence) of the first page that a sequence of ``new_length`` still reads."""
        if g.request.window is None:
            return 0
        # the oldest position any row of the step can see is (first new position) - window + 1;
        # pages are dropped at commit, by the length after the step
        return max(0, new_length - g.request.window) // self.page_size

    def pages_needed(self, s: int, n_new: int) -> List[int]:
        """Pages per group that ``reserve(s, n_new)`` would take."""
        slot = self._slot(s)
        out = []
        for gi, g in enumerate(self.groups):
            first = slot.length // self.page_size
            last = (slot.length + n_new - 1) // self.page_size
            out.append(sum(1 for p in range(first, last + 1) if p not in slot.pages[gi]))
        return out

    def reserve(self, steps: Sequence[Tuple[int, int]]) -> None:
        """Make room for ``n_new`` more tokens in each ``(slot, n_new)``; all or nothing."""
        need = [0] * len(self.groups)
        seen = set()
        for s, n_new in steps:
            if s in seen:
                raise CacheError(f"slot {s} appears twice in one step")
            seen.add(s)
            slot = self._slot(s)
            if n_new <= 0:
                raise CacheError(f"slot {s}: a step must bring at least one token")
            if slot.length + n_new > self.max_seq_len:
                raise CacheFull(f"slot {s}: {slot.length} + {n_new} tokens exceed the longest sequence "
                                f"the cache was sized for ({self.max_seq_len})")
            for gi, n in enumerate(self.pages_needed(s, n_new)):
                need[gi] += n
        for gi, g in enumerate(self.groups):
            if need[gi] > len(g.free):
                raise CacheFull(f"cache group {gi} needs {need[gi]} more pages of {self.page_size} tokens, "
                                f"{len(g.free)} are free")
        for s, n_new in steps:
            slot = self._slots[s]
            for gi, g in enumerate(self.groups):
                first = slot.length // self.page_size
                last = (slot.length + n_new - 1) // self.page_size
                self._ensure_width(last + 1)
                for p in range(first, last + 1):
                    if p not in slot.pages[gi]:
                        page = g.free.pop()
                        slot.pages[gi][p] = page
                        self.tables[gi][s, p] = page

    def commit(self, steps: Sequence[Tuple[int, int]]) -> None:
        """The step ran: lengths grow, and windowed groups give back pages that left the window."""
        for s, n_new in steps:
            slot = self._slot(s)
            slot.length += n_new
            for gi, g in enumerate(self.groups):
                if g.request.window is None:
                    continue
                keep_from = self._first_needed_page(g, slot.length)
                for p in [p for p in slot.pages[gi] if p < keep_from]:
                    g.free.append(slot.pages[gi].pop(p))
                    self.tables[gi][s, p] = 0

    def _ensure_width(self, width: int) -> None:
        if width > self.table_width:
            new = max(width, 2 * self.table_width)
            for gi, t in enumerate(self.tables):
                grown = np.zeros((self.n_slots, new), dtype=np.int32)
                grown[:, :self.table_width] = t
                self.tables[gi] = grown
            self.table_width = new

    def block_table(self, gi: int, slots: Sequence[int], width: int) -> np.ndarray:
        return self.tables[gi][np.asarray(slots, dtype=np.int64), :width]

    def free_pages(self, gi: int = 0) -> int:
        return len(self.groups[gi].free)

    # ------------------------------------------------------------------ invariants
    def check(self) -> None:
        """Raise if a page or slot is lost, held twice or freed twice."""
        for gi, g in enumerate(self.groups):
            held = []
            for si, slot in enumerate(self._slots):
                if not slot.live and slot.pages[gi]:
                    raise CacheError(f"slot {si} is free but still holds pages of group {gi}")
                held.extend(slot.pages[gi].values())
            everything = sorted(held + g.free)
            if everything != list(range(1, g.n_pages)):
                raise CacheError(f"group {gi}: pages are lost or duplicated "
                                 f"({len(held)} held + {len(g.free)} free of {g.n_pages - 1})")
        live = [i for i, s in enumerate(self._slots) if s.live]
        if sorted(live + self._free_slots) != list(range(self.n_slots)):
            raise CacheError("a slot is lost, or both free and live")


class StatePool:
    """Fixed-size per-sequence state: ``[n_slots, *shape]`` per schedule entry that asked for it."""

    def __init__(self, requests: Dict[int, StateRequest], n_slots: int, device: Optional[torch.device] = None):
        self.n_slots = n_slots
        self.tensors: Dict[int, torch.Tensor] = {
            entry: torch.zeros((n_slots, *req.shape), dtype=req.dtype, device=device)
            for entry, req in requests.items()
        }

    def reset(self, slot: int) -> None:
        for t in self.tensors.values():
            t[slot].zero_()

    def of(self, entry: int) -> Optional[torch.Tensor]:
        return self.tensors.get(entry)
