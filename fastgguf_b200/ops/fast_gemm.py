"""bfloat16 tensor-core contractions (tcgen05 / TMA).

``plan_for_weight`` returns an object whose ``run`` either performs the contraction or returns
None when the sizes are outside what the fast kernel takes (a reduction length that is no
multiple of 8, unaligned rows), in which case the caller uses the plain kernel.

With few rows (decode) and few weight tiles the kernel splits the reduction over a thread-block
cluster and sums the partial tiles through distributed shared memory; it needs no scratch memory.
"""
from __future__ import annotations

from ctypes import c_int, c_void_p
from typing import Optional

import torch

from .lib import KernelError, check, lib, ptr, register_signatures, stream

EPI_BF16, EPI_F32, EPI_ADD_F32, EPI_SILU_MUL = 0, 1, 2, 3
_BAD_SIZE = 10002

register_signatures("tc", {
    "fg_gemm_tc": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p],
    "fg_gemm_tc_error": [],
})


def pipeline_error() -> int:
    """0, or the code of the first bounded wait that ran out since the last call (clears it)."""
    return int(lib("tc").fg_gemm_tc_error())


def gemm_tc(a: torch.Tensor, w: torch.Tensor, *, out: Optional[torch.Tensor] = None,
            out_dtype: Optional[torch.dtype] = None, accumulate: bool = False, silu: bool = False,
            force_splits: int = 0) -> Optional[torch.Tensor]:
    """out[m, n] (+)= sum_k a[m, k] w[n, k] on the tensor cores; None if the sizes are refused.

    ``silu=True``: ``w`` is [2F, K] with gate and up interleaved in blocks of 64 rows (see
    ``interleave_gate_up``) and the result is ``silu(a gate^T) * (a up^T)`` as bfloat16 [M, F].
    """
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError("gemm_tc takes bfloat16 operands")
    M, K = a.shape
    rows, K2 = w.shape
    if K != K2:
        raise KernelError(f"gemm_tc: a is [{M}, {K}] but w is [{rows}, {K2}]")
    if a.stride(1) != 1 or w.stride(1) != 1:
        raise KernelError("gemm_tc: the reduction dimension must be contiguous in both operands")
    if silu:
        N, epi, dt = rows // 2, EPI_SILU_MUL, torch.bfloat16
        if rows % 128 or accumulate:
            raise KernelError("gemm_tc: the silu epilogue needs w = [2F, K] with F a multiple of 64, and no accumulation")
    else:
        N = rows
        if accumulate:
            epi, dt = EPI_ADD_F32, torch.float32
        else:
            dt = out_dtype or (out.dtype if out is not None else torch.bfloat16)
            if dt == torch.bfloat16:
                epi = EPI_BF16
            elif dt == torch.float32:
                epi = EPI_F32
            else:
                raise KernelError(f"gemm_tc: cannot write {dt}")
    if out is None:
        if accumulate:
            raise KernelError("gemm_tc: accumulate needs the tensor to accumulate into")
        out = torch.empty((M, N), dtype=dt, device=a.device)
    if out.shape != (M, N) or out.stride(1) != 1 or out.dtype != dt:
        raise KernelError(f"gemm_tc: out must be [{M}, {N}] {dt} with contiguous rows")
    code = lib("tc").fg_gemm_tc(ptr(a), a.stride(0), ptr(w), w.stride(0), ptr(out), out.stride(0), epi,
                                M, rows, K, int(force_splits), stream())
    if code == _BAD_SIZE:
        return None
    check(code, "gemm_tc")
    return out


class _Plan:
    def __init__(self, weight: torch.Tensor):
        self.weight = weight

    def run(self, a, out=None, out_dtype=None, accumulate=False):
        return gemm_tc(a, self.weight, out=out, out_dtype=out_dtype, accumulate=accumulate)

    def run_silu(self, a):
        return gemm_tc(a, self.weight, silu=True)


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """[2F, K]: blocks of 64 gate rows followed by the 64 up rows of the same features."""
    F, K = gate.shape
    if F % 64:
        raise KernelError("interleave_gate_up: the feed-forward width must be a multiple of 64")
    return torch.stack([gate.view(F // 64, 64, K), up.view(F // 64, 64, K)], dim=1).reshape(2 * F, K).contiguous()


def plan_for_weight(weight: torch.Tensor) -> Optional[_Plan]:
    """A plan for a bfloat16 weight on a CUDA device whose rows TMA can address; else None."""
    if weight.dtype != torch.bfloat16 or not weight.is_cuda:
        return None
    if weight.shape[1] % 8 or weight.stride(0) % 8 or weight.data_ptr() % 16 or weight.stride(1) != 1:
        return None
    return _Plan(weight)
