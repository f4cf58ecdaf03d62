"""The device-side description of one step: which rows belong to which sequence, at which
position, with which pages.

A step is a list of ``(slot, tokens, want)``: every sequence brings one or more next tokens
(all prompts of a batch in the first step, one token each afterwards - but any mix is legal)
and names the places among them whose logits it wants.  Rows are laid out sequence after
sequence.  All integer inputs of a step travel to the device in ONE copy from pinned memory;
the tensors below are views into that buffer.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import numpy as np
import torch


@dataclass
class StepEntry:
    slot: int
    tokens: Sequence[int]
    want: Sequence[int] = ()


@dataclass
class Batch:
    n_seq: int
    n_rows: int
    tokens: torch.Tensor          # [M] int32 token ids
    positions: torch.Tensor       # [M] int32 position of each row in its sequence
    row_seq: torch.Tensor         # [M] int32 index of the row's sequence within the step
    cu_rows: torch.Tensor         # [n_seq + 1] int32 first row of each sequence
    seq_start: torch.Tensor       # [n_seq] int32 length of each sequence before the step
    slots: torch.Tensor           # [n_seq] int32 cache / state slot of each sequence
    want_rows: Optional[torch.Tensor]   # [n_want] int32 rows whose logits are wanted
    block_tables: List[torch.Tensor]    # per cache group: [n_seq, width] int32 page ids
    n_want: int = 0
    max_new: int = 1              # most rows any sequence brings
    max_len: int = 1              # longest sequence after the step
    single_token: bool = True     # every sequence brings exactly one token (a decode step)
    want_all: bool = False        # the wanted rows are all rows, in order (the head may take the rows as they are)
    host_cu_rows: List[int] = field(default_factory=list)
    host_seq_start: List[int] = field(default_factory=list)


def validate_entries(entries: Sequence[StepEntry], vocab_size: int) -> None:
    if not entries:
        raise ValueError("a step needs at least one sequence")
    for e in entries:
        if len(e.tokens) == 0:
            raise ValueError(f"slot {e.slot}: a step must bring at least one token")
        for t in e.tokens:
            if not (0 <= int(t) < vocab_size):
                raise ValueError(f"slot {e.slot}: token id {t} lies outside the vocabulary [0, {vocab_size})")
        for w in e.want:
            if not (0 <= int(w) < len(e.tokens)):
                raise ValueError(f"slot {e.slot}: wanted place {w} is not among its {len(e.tokens)} tokens")


def build_batch(entries: Sequence[StepEntry], cache, device: torch.device) -> Batch:
    """Pack the step's integers, copy them once, and slice the views.  The cache must already
    hold pages for the new tokens (``cache.reserve``)."""
    n_seq = len(entries)
    lens = [len(e.tokens) for e in entries]
    M = sum(lens)
    starts = [cache.length(e.slot) for e in entries]
    cu = np.zeros(n_seq + 1, dtype=np.int32)
    np.cumsum(lens, out=cu[1:])
    tokens = np.concatenate([np.asarray(e.tokens, dtype=np.int32) for e in entries])
    positions = np.concatenate([np.arange(s, s + n, dtype=np.int32) for s, n in zip(starts, lens)])
    row_seq = np.repeat(np.arange(n_seq, dtype=np.int32), lens)
    want = np.asarray([cu[i] + int(w) for i, e in enumerate(entries) for w in e.want], dtype=np.int32)
    slots = np.asarray([e.slot for e in entries], dtype=np.int32)
    max_len = max(s + n for s, n in zip(starts, lens))
    width = (max_len + cache.page_size - 1) // cache.page_size
    tables = [cache.block_table(gi, slots, width).reshape(-1) for gi in range(len(cache.groups))]
    parts = [tokens, positions, row_seq, cu, np.asarray(starts, dtype=np.int32), slots, want, *tables]
    # keep every view 16-byte aligned so kernels may use vector loads on them
    offs, total = [], 0
    for p in parts:
        offs.append(total)
        total += (p.size + 3) // 4 * 4
    host = torch.empty(max(total, 4), dtype=torch.int32, pin_memory=device.type == "cuda")
    hn = host.numpy()
    for p, o in zip(parts, offs):
        hn[o:o + p.size] = p
    dev = host.to(device, non_blocking=True)

    def view(i):
        return dev[offs[i]:offs[i] + parts[i].size]

    return Batch(
        n_seq=n_seq, n_rows=M, tokens=view(0), positions=view(1), row_seq=view(2), cu_rows=view(3),
        seq_start=view(4), slots=view(5), want_rows=view(6) if want.size else None,
        block_tables=[view(7 + gi).view(n_seq, width) for gi in range(len(tables))],
        n_want=int(want.size), max_new=max(lens), max_len=max_len, single_token=all(n == 1 for n in lens),
        want_all=bool(want.size == M and np.array_equal(want, np.arange(M, dtype=np.int32))),
        host_cu_rows=cu.tolist(), host_seq_start=starts,
    )
