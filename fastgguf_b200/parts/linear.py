"""A weight matrix [out, in] and the choice of contraction kernel for it.

``y = W x`` with no bias, W row-major [out, in] as in the checkpoint and as the reference
keeps it (fastgguf.c:2582-2585, ``tensor_rows`` :4166).  The reference picks a kernel by tensor
type and batch size inside ``matvec``/``matmul`` (fastgguf.c:2575-2622, 3004-3093); here the
choice is by dtype, row count and alignment:

* float32 operands, or sizes the fast kernels refuse -> the plain FMA kernel (any size);
* bfloat16 with few rows (decode) -> the weight-streaming tensor-core kernel with split-K;
* bfloat16 with many rows (prefill) -> the tiled tcgen05/TMA kernel.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops


class Linear:
    def __init__(self, weight: torch.Tensor):
        if weight.dim() != 2 or weight.stride(1) != 1:
            raise ValueError("Linear: weight must be [out, in] with contiguous rows")
        self.weight = weight
        self.out_features, self.in_features = weight.shape
        self._fast = None
        if weight.dtype == torch.bfloat16 and weight.is_cuda:
            from ..ops import fast_gemm
            self._fast = fast_gemm.plan_for_weight(weight)

    def rows(self, start: int, stop: int) -> "Linear":
        """The sub-matrix of output rows [start, stop) (shares storage)."""
        return Linear(self.weight[start:stop])

    def forward(self, a, out: Optional[torch.Tensor] = None, out_dtype: Optional[torch.dtype] = None,
                accumulate: bool = False, emit_norm=None):
        """out[m, n] (+)= sum_k a[m, k] W[n, k].  ``accumulate`` adds into a float32 ``out``.

        ``a`` may be a ``DeferredNorm`` (rows x * w whose 1/rms the tensor-core kernel applies).
        ``emit_norm`` (a norm part with ``weight``, ``eps``; needs ``accumulate``): the call returns
        ``(out, DeferredNorm or None)`` - the next norm started from the updated ``out`` when the
        tensor-core kernel ran, None when the plain kernel did."""
        from ..ops.fast_gemm import DeferredNorm
        deferred = a if isinstance(a, DeferredNorm) else None
        if self._fast is not None and (deferred is not None or a.dtype == torch.bfloat16):
            res = self._fast.run(deferred.xw if deferred is not None else a, out=out, out_dtype=out_dtype,
                                 accumulate=accumulate, deferred=deferred,
                                 emit_norm_weight=emit_norm.weight if emit_norm is not None else None,
                                 emit_eps=emit_norm.eps if emit_norm is not None else 0.0)
            if res is not None:
                return res
        if deferred is not None:
            a = deferred.materialize()
        res = ops.gemm_generic(a, self.weight, out=out, out_dtype=out_dtype, accumulate=accumulate)
        return (res, None) if emit_norm is not None else res
