"""Parts a decoder is put together from; see ``parts.base`` for the interfaces."""
from .base import (Block, CacheRequest, FeedForward, LayerIO, Mixer, Norm, Part, PositionEncoding, Runtime,
                   StateRequest, TensorSpec, lookup, register_block, register_feed_forward, register_mixer,
                   register_norm, register_position_encoding)

_builtin_loaded = False


def _load_builtin() -> None:
    global _builtin_loaded
    if not _builtin_loaded:
        _builtin_loaded = True
        from . import attention, block, mlp, norm, rope  # noqa: F401  (each registers its kinds)


__all__ = [
    "Block", "CacheRequest", "FeedForward", "LayerIO", "Mixer", "Norm", "Part", "PositionEncoding", "Runtime",
    "StateRequest", "TensorSpec", "lookup", "register_block", "register_feed_forward", "register_mixer",
    "register_norm", "register_position_encoding",
]
