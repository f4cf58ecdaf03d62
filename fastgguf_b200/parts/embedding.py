"""TokenEmbedding(vocab_size, hidden_size) and LMHead(vocab_size, hidden_size, tied).

Reference: ``read_embedding`` copies row ``token`` of ``token_embd`` into the residual stream
with scale 1 for Llama (fastgguf.c:4576-4581, :4652, :4219); the head is ``output.weight`` or,
when that tensor is absent, the embedding table again (:4269-4270); logits are float
(:4900).  Here tied-ness comes from the configuration, and a tied head shares the embedding's
storage.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import ops
from .base import Part, Runtime, TensorSpec
from .linear import Linear


class TokenEmbedding(Part):
    def __init__(self, runtime: Runtime, vocab_size: int, hidden_size: int):
        super().__init__(runtime)
        self.vocab_size, self.hidden_size = vocab_size, hidden_size
        self.weight: Optional[torch.Tensor] = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {"weight": TensorSpec((self.vocab_size, self.hidden_size))}

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.weight = tensors["weight"].contiguous()

    def forward(self, tokens: torch.Tensor, emit_norm=None):
        """The float32 residual stream [M, E]; with ``emit_norm`` (a deferrable norm) also that
        norm started from it: returns ``(x, DeferredNorm or None)``."""
        if emit_norm is None:
            return ops.embed_gather(self.weight, tokens)
        if self.runtime.dtype == torch.bfloat16 and self.weight.is_cuda:
            return ops.embed_gather_norm(self.weight, tokens, emit_norm.weight, emit_norm.eps)
        return ops.embed_gather(self.weight, tokens), None


class LMHead(Part):
    #: ``forward`` also takes rows whose RMSNorm was started by the contraction before (x * w and partial sums of squares)
    supports_deferred_norm = True

    def __init__(self, runtime: Runtime, vocab_size: int, hidden_size: int):
        super().__init__(runtime)
        self.vocab_size, self.hidden_size = vocab_size, hidden_size
        self.linear: Optional[Linear] = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {"weight": TensorSpec((self.vocab_size, self.hidden_size))}

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.linear = Linear(tensors["weight"])

    def forward(self, xn) -> torch.Tensor:
        """Float32 logits [rows, vocab] of normalized rows (a tensor, or a ``DeferredNorm``)."""
        return self.linear.forward(xn, out_dtype=torch.float32)
