"""The data that describes a model, as Python objects: which parts, in which layers, run in which order.

The host works from the JSON form (``csrc/fastgguf_parts.h`` describes it); these classes build and read it:

* every part is a :class:`PartSpec` - a registered kind name, its sizes and constants as parameters, and
  the checkpoint names of its tensors;
* every layer names its own block arrangement, mixer, feed-forward and norms, so one model can mix kinds
  layer by layer;
* the order in which layers run is the list ``schedule``: an entry may name a layer that already ran (shared
  weights, a cache of its own) or read the cache of an earlier entry instead of writing one.

The reference expresses the same choices as flags and optional per-layer tensors on one struct (``is_swa[]``,
``kv_donor[]``, optional norms; fastgguf.c:4064-4100) and a fixed ``for il < n_layer`` loop (:4674).
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

    def to_json(self) -> dict:
        def conv(v):
            return v.to_json() if isinstance(v, PartSpec) else v
        return {"kind": self.kind, "params": {k: conv(v) for k, v in self.params.items()}, "tensors": dict(self.tensors)}

    @classmethod
    def from_json(cls, j: dict) -> "PartSpec":
        params = {k: (cls.from_json(v) if isinstance(v, dict) and "kind" in v and "params" in v else v)
                  for k, v in (j.get("params") or {}).items()}
        return cls(j["kind"], params, dict(j.get("tensors") or {}))


@dataclass
class LayerSpec:
    block: str                     # arrangement kind, e.g. "prenorm"
    mixer: PartSpec
    feed_forward: PartSpec
    mixer_norm: PartSpec
    feed_forward_norm: PartSpec

    def to_json(self) -> dict:
        return {"block": self.block, "mixer": self.mixer.to_json(), "feed_forward": self.feed_forward.to_json(),
                "mixer_norm": self.mixer_norm.to_json(), "feed_forward_norm": self.feed_forward_norm.to_json()}


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

    def to_json(self) -> dict:
        return {
            "hidden_size": self.hidden_size, "vocab_size": self.vocab_size, "max_positions": self.max_positions,
            "embedding": self.embedding.to_json(), "final_norm": self.final_norm.to_json(), "head": self.head.to_json(),
            "layers": [l.to_json() for l in self.layers],
            "schedule": [{"layer": r.layer, "cache_from": r.cache_from} for r in self.schedule],
            "stop_token_ids": list(self.stop_token_ids), "ignored_tensors": list(self.ignored_tensors),
        }

    @classmethod
    def from_json(cls, j: dict) -> "ModelSpec":
        P = PartSpec.from_json
        return cls(
            hidden_size=j["hidden_size"], vocab_size=j["vocab_size"], max_positions=j["max_positions"],
            embedding=P(j["embedding"]), final_norm=P(j["final_norm"]), head=P(j["head"]),
            layers=[LayerSpec(l["block"], P(l["mixer"]), P(l["feed_forward"]), P(l["mixer_norm"]), P(l["feed_forward_norm"]))
                    for l in j["layers"]],
            schedule=[RunSpec(r["layer"], r.get("cache_from")) for r in j["schedule"]],
            stop_token_ids=tuple(j.get("stop_token_ids") or ()), ignored_tensors=tuple(j.get("ignored_tensors") or ()),
        )
