"""Interfaces of the parts a decoder layer is put together from, and their registries.

Roles: *norm*, *position encoding*, *mixer* (attention here), *feed-forward* and the *block*
that arranges them.  A part is built from a :class:`~fastgguf_b200.engine.spec.PartSpec`: its
kind is looked up in the registry of its role and its sizes and constants arrive as keyword
parameters.  No part knows which model it is in; a new kind is one ``register_*`` call away
(tests register toy kinds without touching the framework).

What every part provides
    ``tensor_specs()``  local tensor name -> :class:`TensorSpec` (shape, float or integer, how
                        random weights are drawn); the loader checks the checkpoint against it.
    ``load(tensors)``   receives its tensors on the device, in the engine's dtype policy.

Norm            ``forward(x, rows=None) -> act``     x: [M, E] f32 residual stream; returns the
                                                      engine's activation dtype; ``rows`` picks rows.
PositionEncoding ``prepare(max_positions)``           builds its device tables once.
Mixer           ``cache_request()``                   -> CacheRequest or None (keys/values it keeps)
                ``state_request()``                   -> StateRequest or None (fixed-size state)
                ``forward(xn, batch, io, residual)``  adds its output into ``residual`` ([M, E] f32)
FeedForward     ``forward(xn, batch, residual)``      adds its output into ``residual``
Block           ``forward(x, batch, io, pending, next_norm)``  runs norm/mixer/norm/feed-forward on ``x`` in place

Optional protocol (an optimisation, never needed for correctness): a norm with ``deferrable = True``
(and ``weight``, ``eps``) can be *started* by the contraction that produces its input and *finished*
by the contraction that consumes it; mixers and feed-forwards that set
``supports_deferred_norm = True`` accept a ``DeferredNorm`` as ``xn`` and an ``emit_norm=`` keyword.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, Optional, Tuple

import torch


@dataclass(frozen=True)
class TensorSpec:
    shape: Tuple[int, ...]
    #: "float" tensors follow the engine dtype policy; "int" tables are kept as int32
    kind: str = "float"
    #: how random weights are drawn: ("normal", std) or ("one_plus_normal", std)
    init: Tuple[str, float] = ("normal", 0.02)


@dataclass(frozen=True)
class CacheRequest:
    """Keys and values a mixer keeps per position.  ``window`` None keeps every position; an
    integer keeps the last ``window`` positions.  Requests that agree in all fields share a
    cache group (one page table, one pool per schedule entry)."""

    n_kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class StateRequest:
    """Per-sequence state of fixed size, zeroed when a sequence takes its slot."""

    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclass
class Runtime:
    """What parts need from the engine: the device and the activation/weight dtype."""

    device: torch.device
    dtype: torch.dtype            # torch.bfloat16 (serving) or torch.float32 (true 32-bit path)


@dataclass
class LayerIO:
    """What one schedule entry owns or borrows: cache pools and state rows."""

    group: Optional[int] = None               # cache group index (block table to use)
    k_pool: Optional[torch.Tensor] = None     # [pages, KV, page, hd]
    v_pool: Optional[torch.Tensor] = None
    write_cache: bool = True                  # False: the cache belongs to an earlier entry
    state: Optional[torch.Tensor] = None      # [n_slots, *StateRequest.shape]


class Part:
    def __init__(self, runtime: Runtime):
        self.runtime = runtime

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {}

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        pass


class Norm(Part):
    def forward(self, x: torch.Tensor, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        raise NotImplementedError


class PositionEncoding(Part):
    def prepare(self, max_positions: int) -> None:
        raise NotImplementedError


class Mixer(Part):
    def cache_request(self) -> Optional[CacheRequest]:
        return None

    def state_request(self) -> Optional[StateRequest]:
        return None

    def forward(self, xn: torch.Tensor, batch, io: LayerIO, residual: torch.Tensor) -> None:
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, xn: torch.Tensor, batch, residual: torch.Tensor) -> None:
        raise NotImplementedError


class Block:
    """An arrangement of a mixer, a feed-forward and their norms around the residual stream."""

    def __init__(self, mixer: Mixer, feed_forward: FeedForward, mixer_norm: Norm, feed_forward_norm: Norm):
        self.mixer, self.feed_forward = mixer, feed_forward
        self.mixer_norm, self.feed_forward_norm = mixer_norm, feed_forward_norm

    def forward(self, x: torch.Tensor, batch, io: LayerIO, pending=None, next_norm=None):
        """Run the block on ``x`` in place.  ``pending`` / ``next_norm`` / the return value let a
        block hand a started norm to the next one (see ``PreNormBlock``); a block may ignore them
        and return None."""
        raise NotImplementedError


# ---------------------------------------------------------------------------------------
# registries, one per role
_REGISTRIES: Dict[str, Dict[str, Callable]] = {
    "norm": {}, "position": {}, "mixer": {}, "feed_forward": {}, "block": {},
}


def _register(role: str, kind: str, factory: Callable) -> None:
    _REGISTRIES[role][kind] = factory


def register_norm(kind: str, factory: Callable) -> None:
    _register("norm", kind, factory)


def register_position_encoding(kind: str, factory: Callable) -> None:
    _register("position", kind, factory)


def register_mixer(kind: str, factory: Callable) -> None:
    _register("mixer", kind, factory)


def register_feed_forward(kind: str, factory: Callable) -> None:
    _register("feed_forward", kind, factory)


def register_block(kind: str, factory: Callable) -> None:
    _register("block", kind, factory)


def lookup(role: str, kind: str) -> Callable:
    from . import _load_builtin
    _load_builtin()
    try:
        return _REGISTRIES[role][kind]
    except KeyError:
        raise KeyError(f"no {role} of kind '{kind}' is registered "
                       f"(registered: {', '.join(sorted(_REGISTRIES[role])) or 'none'})") from None
