"""PreNormBlock: ``x += mixer(norm1(x)); x += feed_forward(norm2(x))``.

Reference: the norm stands before attention (fastgguf.c:4686-4687) and before the feed-forward
(:4865-4866); both residual sums add the projection onto the un-normalized input (:4862, :4880).
The residual stream ``x`` is float32 and is updated in place by the parts' output projections.
"""
from __future__ import annotations

from .base import Block, LayerIO, register_block


class PreNormBlock(Block):
    def forward(self, x, batch, io: LayerIO) -> None:
        self.mixer.forward(self.mixer_norm.forward(x), batch, io, x)
        self.feed_forward.forward(self.feed_forward_norm.forward(x), batch, x)


register_block("prenorm", PreNormBlock)
