"""SwiGLU(hidden_size, d_ff): ``down( silu(gate x) * (up x) )``.

Reference (fastgguf.c): gate and up in one fused pass (:4870-4872), ``silu(z) = z / (1 + exp(-z))``
(:3118) times up (:4876), down projection added onto the layer's input (:4877-4880).
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import ops
from .base import FeedForward, Runtime, TensorSpec, register_feed_forward
from .linear import Linear


class SwiGLU(FeedForward):
    supports_deferred_norm = True

    def __init__(self, runtime: Runtime, hidden_size: int, d_ff: int):
        super().__init__(runtime)
        self.hidden_size, self.d_ff = hidden_size, d_ff
        self.gate_up: Optional[Linear] = None
        self.down: Optional[Linear] = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        E, F = self.hidden_size, self.d_ff
        return {
            "gate_proj.weight": TensorSpec((F, E)),
            "up_proj.weight": TensorSpec((F, E)),
            "down_proj.weight": TensorSpec((E, F)),
        }

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        g, u = tensors["gate_proj.weight"], tensors["up_proj.weight"]
        dt = g.dtype if g.dtype == u.dtype else torch.float32
        self.fused = None
        if dt == torch.bfloat16 and g.is_cuda and self.d_ff % 64 == 0 and self.hidden_size % 8 == 0:
            from ..ops import fast_gemm
            # gate, up and SiLU-mul in one tensor-core kernel: rows interleaved in blocks of 64
            self.fused = fast_gemm.plan_for_weight(fast_gemm.interleave_gate_up(g, u))
        if self.fused is None:
            self.gate_up = Linear(torch.cat([g.to(dt), u.to(dt)], dim=0).contiguous())
        self.down = Linear(tensors["down_proj.weight"].contiguous())

    def forward(self, xn, batch, residual: torch.Tensor, emit_norm=None):
        from ..ops.fast_gemm import DeferredNorm
        deferred = xn if isinstance(xn, DeferredNorm) else None
        if self.fused is not None:
            t = self.fused.run_silu(deferred.xw if deferred is not None else xn, deferred=deferred)
            if t is None:
                raise ops.KernelError("the fused gate/up kernel refused a shape it was planned for")
        else:
            t = ops.silu_mul(self.gate_up.forward(xn, out_dtype=self.runtime.dtype))
        if emit_norm is None:
            self.down.forward(t, out=residual, accumulate=True)
            return None
        return self.down.forward(t, out=residual, accumulate=True, emit_norm=emit_norm)[1]


register_feed_forward("swiglu", SwiGLU)
