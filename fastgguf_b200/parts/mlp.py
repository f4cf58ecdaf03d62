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
        self.gate_up = Linear(torch.cat([g.to(dt), u.to(dt)], dim=0).contiguous())
        self.down = Linear(tensors["down_proj.weight"].contiguous())

    def forward(self, xn: torch.Tensor, batch, residual: torch.Tensor) -> None:
        t = None
        if self.gate_up._fast is not None and xn.dtype == torch.bfloat16:
            t = self.gate_up._fast.run_silu(xn, self.d_ff)      # gate, up and SiLU-mul in one kernel
        if t is None:
            t = ops.silu_mul(self.gate_up.forward(xn, out_dtype=self.runtime.dtype))
        self.down.forward(t, out=residual, accumulate=True)


register_feed_forward("swiglu", SwiGLU)
