"""bfloat16 tensor-core contractions (tcgen05 / TMA).

``plan_for_weight`` returns an object whose ``run`` either performs the contraction or returns
None when the sizes are outside what the fast kernel takes (a reduction length that is no
multiple of 8, unaligned rows), in which case the caller uses the plain kernel.

With few rows (decode) one kernel serves every projection; with few weight tiles it splits the reduction
over a thread-block cluster, whose CTAs push their partial columns into the owner's shared memory; it
needs no scratch memory.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p
from dataclasses import dataclass
from typing import Optional

import torch

from .lib import KernelError, check, lib, ptr, register_signatures, stream

EPI_BF16, EPI_F32, EPI_ADD_F32, EPI_SILU_MUL = 0, 1, 2, 3
_BAD_SIZE = 10002

register_signatures("tc", {
    "fg_gemm_tc": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                   c_void_p, c_int, c_int, c_float, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p],
    "fg_gemm_tc_ws": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                      c_void_p, c_int, c_int, c_float, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_longlong, c_void_p],
    "fg_gemm_tc_workspace_bytes": [c_int, c_int, c_int, c_int],
    "fg_gemm_tc_error": [],
    "fg_gemm_tc_max_ss_tiles": [c_int],
})


def workspace_bytes(M: int, N: int, K: int, epi: int) -> int:
    """Bytes of scratch memory with which the contraction is split along K (0: it is not split)."""
    fn = lib("tc").fg_gemm_tc_workspace_bytes
    fn.restype = c_longlong
    return int(fn(M, N, K, epi))


@dataclass
class DeferredNorm:
    """An RMSNorm whose 1/rms has not been applied yet: ``xw = bf16(x * weight)`` and partial sums of
    squares of each row of x (``ss[t, m]``, t < tiles).  A tensor-core contraction takes ``xw`` as its
    input and applies 1/sqrt(sum / size + eps) per row in its epilogue; ``materialize`` gives the
    normalised rows to anything else."""

    xw: torch.Tensor              # [M, size] bfloat16
    ss: torch.Tensor              # [>= tiles, M] float32
    tiles: int
    size: int
    eps: float
    x: torch.Tensor               # [M, size] float32: the rows being normalised
    weight: torch.Tensor          # [size] float32: the norm's weight

    def materialize(self) -> torch.Tensor:
        """The normalised rows, by the RMSNorm kernel (for consumers that cannot apply 1/rms themselves)."""
        from . import rmsnorm
        return rmsnorm(self.x, self.weight, self.eps, torch.bfloat16)


def pipeline_error() -> int:
    """0, or the code of the first bounded wait that ran out since the last call (clears it)."""
    return int(lib("tc").fg_gemm_tc_error())


def gemm_tc(a: torch.Tensor, w: torch.Tensor, *, out: Optional[torch.Tensor] = None,
            out_dtype: Optional[torch.dtype] = None, accumulate: bool = False, silu: bool = False,
            force_splits: int = 0, deferred: Optional["DeferredNorm"] = None,
            emit_norm_weight: Optional[torch.Tensor] = None, emit_eps: float = 0.0, split_k: bool = True):
    """out[m, n] (+)= sum_k a[m, k] w[n, k] on the tensor cores; None if the sizes are refused.

    ``silu=True``: ``w`` is [2F, K] with gate and up interleaved in blocks of 64 rows (see
    ``interleave_gate_up``) and the result is ``silu(a gate^T) * (a up^T)`` as bfloat16 [M, F].
    ``deferred``: ``a`` is ``deferred.xw`` and the rows' 1/rms is applied in the epilogue.
    ``emit_norm_weight`` (with ``accumulate``): also start the next RMSNorm from the updated ``out``;
    the call then returns ``(out, DeferredNorm)``.
    ``split_k=False``: no scratch memory is offered, so a contraction of few output tiles is not split along K.
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
    ss_in, ss_tiles, ss_size, ss_eps = None, 0, 1, 0.0
    if deferred is not None:
        ss_in, ss_tiles, ss_size, ss_eps = deferred.ss, deferred.tiles, deferred.size, deferred.eps
    xw_out = ss_out = None
    tiles_out = ctypes.c_int(0)
    if emit_norm_weight is not None:
        if not accumulate or emit_norm_weight.dtype != torch.float32 or emit_norm_weight.numel() != N:
            raise KernelError("gemm_tc: emitting a norm needs the residual-add epilogue and a float32 weight [N]")
        xw_out = torch.empty((M, N), dtype=torch.bfloat16, device=a.device)
        ss_out = torch.empty((int(lib("tc").fg_gemm_tc_max_ss_tiles(N)), M), dtype=torch.float32, device=a.device)
    need = workspace_bytes(M, rows, K, epi) if split_k and not force_splits else 0
    scratch = torch.empty(need, dtype=torch.uint8, device=a.device) if need else None
    code = lib("tc").fg_gemm_tc_ws(ptr(a), a.stride(0), ptr(w), w.stride(0), ptr(out), out.stride(0), epi,
                                   M, rows, K, int(force_splits), ptr(ss_in), ss_tiles, ss_size, float(ss_eps),
                                   ptr(emit_norm_weight), ptr(xw_out), ptr(ss_out), ctypes.byref(tiles_out),
                                   ptr(scratch), need, stream())
    if code == _BAD_SIZE:
        return None
    check(code, "gemm_tc")
    if emit_norm_weight is not None:
        return out, DeferredNorm(xw_out, ss_out, int(tiles_out.value), N, float(emit_eps), out, emit_norm_weight)
    return out


class _Plan:
    def __init__(self, weight: torch.Tensor):
        self.weight = weight

    def run(self, a, out=None, out_dtype=None, accumulate=False, deferred=None, emit_norm_weight=None, emit_eps=0.0):
        return gemm_tc(a, self.weight, out=out, out_dtype=out_dtype, accumulate=accumulate, deferred=deferred,
                       emit_norm_weight=emit_norm_weight, emit_eps=emit_eps)

    def run_silu(self, a, deferred=None):
        return gemm_tc(a, self.weight, silu=True, deferred=deferred)


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
