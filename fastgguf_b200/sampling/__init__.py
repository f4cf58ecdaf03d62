"""Next-token selection: parameters, per-sequence state on the device, and the kernel call.

Options and defaults are the reference's chat sampler (fastgguf.c:6976-6982):
``temp 1.0`` (0 = greedy), ``top_k 64`` (0 = off), ``top_p 0.95``, ``repeat_penalty 1.0``
(1 = off), ``repeat_last_n 64``, ``seed`` (0 = take one from the clock, :5232-5233).  The order
of operations is ``sample_next`` (:4008-4056); see ``csrc/sampling.cu``.

Each sequence has a state row of its own - an xorshift64* generator (:3334-3339) and the ring of
its recent tokens for the repeat penalty - so what a sequence draws does not depend on its
batch-mates.  The first request of a call starts from ``seed`` itself, as the reference's single
conversation does; request i > 0 starts from a mix of (seed, i).
"""
from __future__ import annotations

import time
from dataclasses import dataclass
from typing import Optional, Sequence

import torch

from .. import ops

MASK64 = (1 << 64) - 1


@dataclass(frozen=True)
class SamplingParams:
    temp: float = 1.0
    top_k: int = 64
    top_p: float = 0.95
    repeat_penalty: float = 1.0
    repeat_last_n: int = 64
    seed: int = 0

    def validate(self) -> None:
        if self.top_k > 1024:
            raise ValueError(f"top_k {self.top_k} exceeds 1024, the most the sampler takes (0 turns top-k off)")
        if self.repeat_last_n < 0:
            raise ValueError("repeat_last_n cannot be negative")

    @property
    def greedy(self) -> bool:
        return self.temp <= 0.0

    @property
    def penalizes(self) -> bool:
        return self.repeat_penalty > 0.0 and self.repeat_penalty != 1.0 and self.repeat_last_n > 0


def resolve_seed(seed: int) -> int:
    """0 means "from the clock"; the state of xorshift64* must never be zero (fastgguf.c:5232-5233)."""
    if seed == 0:
        seed = (int(time.time()) * 0x9E3779B97F4A7C15 ^ time.perf_counter_ns() // 1000) & MASK64
    return (seed & MASK64) or 0x9E3779B97F4A7C15


def request_seed(seed: int, index: int) -> int:
    """Generator state of request ``index`` of a call seeded with ``seed`` (already resolved)."""
    if index == 0:
        return seed
    z = (seed + index * 0x9E3779B97F4A7C15) & MASK64           # splitmix64 finaliser
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & MASK64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & MASK64
    z ^= z >> 31
    return z or 0x9E3779B97F4A7C15


def _as_i64(v: int) -> int:
    return v - (1 << 64) if v >= (1 << 63) else v


class Sampler:
    """Device state for ``n_rows`` sequences (one row per cache slot, plus a spare row that
    padded rows of a fixed-shape step use)."""

    def __init__(self, params: SamplingParams, n_rows: int, stop_ids: Sequence[int], device: torch.device):
        params.validate()
        self.params, self.device = params, device
        self.n_rows = n_rows + 1
        self.spare_row = n_rows
        self.rng = torch.full((self.n_rows,), _as_i64(0x9E3779B97F4A7C15), dtype=torch.int64, device=device)
        self.hist_cap = max(1, params.repeat_last_n)
        self.use_hist = params.penalizes
        self.hist = torch.zeros((self.n_rows, self.hist_cap), dtype=torch.int32, device=device) if self.use_hist else None
        self.hist_count = torch.zeros((self.n_rows,), dtype=torch.int32, device=device) if self.use_hist else None
        self.stop_ids = (torch.tensor(list(stop_ids), dtype=torch.int32, device=device) if stop_ids else None)

    def begin(self, row: int, state: int, prompt: Sequence[int]) -> None:
        """Give a sequence its generator state and the tail of its prompt as history."""
        self.rng[row] = _as_i64(state)
        if self.use_hist:
            tail = list(prompt)[-self.hist_cap:]
            self.hist_count[row] = len(tail)
            if tail:
                self.hist[row, :len(tail)] = torch.tensor(tail, dtype=torch.int32, device=self.device)

    def sample(self, logits: torch.Tensor, rows: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """One token per row of ``logits`` ([B, V] float32); ``rows[b]`` is the state row of sequence b."""
        p = self.params
        return ops.sample(logits, temp=p.temp, top_k=p.top_k, top_p=p.top_p, repeat_penalty=p.repeat_penalty,
                          repeat_last_n=p.repeat_last_n, seq_slot=rows, rng=self.rng, hist=self.hist,
                          hist_count=self.hist_count, stop_ids=self.stop_ids, out=out)
