"""PreNormBlock: ``x += mixer(norm1(x)); x += feed_forward(norm2(x))``.

Reference: the norm stands before attention (fastgguf.c:4686-4687) and before the feed-forward
(:4865-4866); both residual sums add the projection onto the un-normalized input (:4862, :4880).
The residual stream ``x`` is float32 and is updated in place by the parts' output projections.
"""
from __future__ import annotations

import torch

from .base import Block, LayerIO, register_block


class PreNormBlock(Block):
    def forward(self, x, batch, io: LayerIO, pending=None, next_norm=None):
        """``pending``: the mixer norm already started by whoever produced ``x`` (a ``DeferredNorm``);
        ``next_norm``: the norm that will read ``x`` after this block, to be started by the
        feed-forward's last projection.  Both are optional; parts that do not take part get plain
        normalised tensors.  Returns the started ``next_norm`` or None."""
        def can(part):
            return getattr(part, "supports_deferred_norm", False) and self.mixer.runtime.dtype == torch.bfloat16

        xn = pending if (pending is not None and can(self.mixer)) else self.mixer_norm.forward(x)
        started = None
        if can(self.mixer):
            emit = self.feed_forward_norm if (can(self.feed_forward) and getattr(self.feed_forward_norm, "deferrable", False)) else None
            started = self.mixer.forward(xn, batch, io, x, emit_norm=emit)
        else:
            self.mixer.forward(xn, batch, io, x)
        xn2 = started if started is not None else self.feed_forward_norm.forward(x)
        if can(self.feed_forward):
            return self.feed_forward.forward(xn2, batch, x, emit_norm=next_norm)
        self.feed_forward.forward(xn2, batch, x)
        return None


register_block("prenorm", PreNormBlock)
