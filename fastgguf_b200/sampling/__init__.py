"""Next-token selection: the parameters as Python passes them to the host.

Options and defaults are the reference's chat sampler (fastgguf.c:6976-6982): ``temp 1.0`` (0 = greedy),
``top_k 64`` (0 = off), ``top_p 0.95``, ``repeat_penalty 1.0`` (1 = off), ``repeat_last_n 64``, ``seed`` (0 =
take one from the clock, :5232-5233).  The order of operations is ``sample_next`` (:4008-4056); see
``csrc/sampling.cu``.  Each sequence has a state row of its own in the host's ``Sampler`` - an xorshift64*
generator (:3334-3339) and the ring of its recent tokens for the repeat penalty - so what a sequence draws does
not depend on its batch-mates.  The first request of a call starts from ``seed`` itself, as the reference's single
conversation does; request i > 0 starts from a mix of (seed, i).
"""
from __future__ import annotations

from ctypes import byref, c_uint64
from dataclasses import dataclass

from .. import capi

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

    def to_struct(self) -> capi.Sampling:
        self.validate()
        return capi.Sampling(float(self.temp), int(self.top_k), float(self.top_p), float(self.repeat_penalty),
                             int(self.repeat_last_n), int(self.seed) & MASK64)


def resolve_seed(seed: int) -> int:
    """0 means "from the clock"; the state of xorshift64* must never be zero (fastgguf.c:5232-5233)."""
    out = c_uint64()
    capi.check(capi.lib().fg_seed_resolve(int(seed) & MASK64, byref(out)))
    return out.value


def request_seed(seed: int, index: int) -> int:
    """Generator state of request ``index`` of a call seeded with ``seed`` (already resolved)."""
    out = c_uint64()
    capi.check(capi.lib().fg_seed_of_request(int(seed) & MASK64, int(index), byref(out)))
    return out.value
