"""The data that describes a model: which parts, in which layers, run in which order.

An architecture file (``fastgguf_b200/models/*.py``) turns its typed configuration into a
:class:`ModelSpec`.  The spec is plain data:

* every part is a :class:`PartSpec` - a registered kind name, its sizes and constants as
  parameters, and the checkpoint names of its tensors;
* every layer names its own block arrangement, mixer, feed-forward and norms, so one model can
  mix kinds layer by layer;
* the order in which layers run is the list ``schedule``: an entry may name a layer that
  already ran (shared weights, a cache of its own) or read the cache of an earlier entry
  instead of writing one.

The reference expresses the same choices as flags and optional per-layer tensors on one
struct (``is_swa[]``, ``kv_donor[]``, optional norms; fastgguf.c:4064-4100) and a fixed
``for il < n_layer`` loop (fastgguf.c:4674).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple


@dataclass
class PartSpec:
    """A part to build: ``kind`` is looked up in the part registry of its role."""

    kind: str
    params: dict = field(default_factory=dict)
    #: local tensor name of the part -> tensor name in the checkpoint
    tensors: Dict[str, str] = field(default_factory=dict)


@dataclass
class LayerSpec:
    block: str                     # arrangement kind, e.g. "prenorm"
    mixer: PartSpec
    feed_forward: PartSpec
    mixer_norm: PartSpec
    feed_forward_norm: PartSpec


@dataclass
class RunSpec:
    """One entry of the execution order."""

    layer: int
    #: index of an EARLIER schedule entry whose cache this run reads instead of owning one
    cache_from: Optional[int] = None


@dataclass
class ModelSpec:
    hidden_size: int
    vocab_size: int
    max_positions: int
    embedding: PartSpec
    layers: List[LayerSpec]
    schedule: List[RunSpec]
    final_norm: PartSpec
    head: PartSpec
    stop_token_ids: Tuple[int, ...] = ()
    #: regular expressions of checkpoint tensors that may be present without being used
    ignored_tensors: Tuple[str, ...] = ()

    def validate(self) -> None:
        for i, run in enumerate(self.schedule):
            if not (0 <= run.layer < len(self.layers)):
                raise ValueError(f"schedule[{i}] names layer {run.layer}, but there are {len(self.layers)} layers")
            if run.cache_from is not None:
                if not (0 <= run.cache_from < i):
                    raise ValueError(f"schedule[{i}].cache_from must name an earlier entry, got {run.cache_from}")
                if self.schedule[run.cache_from].cache_from is not None:
                    raise ValueError(f"schedule[{i}].cache_from names entry {run.cache_from}, which owns no cache")
