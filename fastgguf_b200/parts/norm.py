"""RMSNorm(size, eps): ``y = x * (1 / sqrt(mean(x^2) + eps)) * w``.

Reference: ``rmsnorm_w`` (fastgguf.c:3100-3105); the weight multiplies directly (no +1), the
multiplication order is x * inv * w.  Statistics are 32-bit here (the reference sums in double).
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import ops
from .base import Norm, Runtime, TensorSpec, register_norm


class RMSNorm(Norm):
    #: a contraction that follows this norm may apply its 1/rms itself (see ``ops.fast_gemm.DeferredNorm``)
    deferrable = True

    def __init__(self, runtime: Runtime, size: int, eps: float):
        super().__init__(runtime)
        self.size, self.eps = int(size), float(eps)
        self.weight: Optional[torch.Tensor] = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {"weight": TensorSpec((self.size,), init=("one_plus_normal", 0.01))}

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        # widening bf16 -> f32 is exact; the kernel reads the weight as f32
        self.weight = tensors["weight"].to(torch.float32).contiguous()

    def forward(self, x: torch.Tensor, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        return ops.rmsnorm(x, self.weight, self.eps, self.runtime.dtype, rows=rows)


register_norm("rmsnorm", RMSNorm)
