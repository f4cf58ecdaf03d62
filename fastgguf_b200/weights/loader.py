"""Weights by tensor name, with one error that says everything that is wrong.

Reference: ``must_tensor`` / ``must_f32`` print ``missing tensor: NAME`` and raise a flag that
is checked after all layers were visited (fastgguf.c:4154-4164, :4387); optional tensors are
looked up with ``tensor_find`` (:4269, :4278); shapes that do not fit the configuration are
errors (:4309-4314, :4330-4335).

dtype policy: in the bfloat16 engine, float tensors stored in 16 bits become bfloat16; a
tensor stored in 32 bits stays float32 (the contraction kernels take mixed operands);
integer tables become int32.  In the float32 engine every float tensor is widened to float32,
which is exact for bfloat16 and float16 sources.
"""
from __future__ import annotations

import json
import os
import re
from typing import Dict, Iterable, List

import torch

from ..parts.base import TensorSpec
from .safetensors_io import SafetensorsError, SafetensorsFile


class WeightError(ValueError):
    """Missing, unexpected or wrongly shaped tensors; the message lists all of them."""

    def __init__(self, where: str, missing: List[str], unexpected: List[str], wrong: List[str]):
        self.missing, self.unexpected, self.wrong = missing, unexpected, wrong
        lines = [f"{where}: the weights do not fit the configuration"]
        if missing:
            lines.append(f"  missing tensors ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            lines.append(f"  unexpected tensors ({len(unexpected)}): " + ", ".join(unexpected))
        if wrong:
            lines.append(f"  wrong shapes or types ({len(wrong)}): " + "; ".join(wrong))
        super().__init__("\n".join(lines))


class TensorSource:
    """Where named tensors come from (a model folder, or tensors already in memory)."""

    def names(self) -> Iterable[str]:
        raise NotImplementedError

    def shape_dtype(self, name: str):
        raise NotImplementedError

    def tensor(self, name: str) -> torch.Tensor:
        raise NotImplementedError

    where = "weights"


class FolderSource(TensorSource):
    """``model.safetensors``, or the shards named by ``model.safetensors.index.json``."""

    def __init__(self, model_dir: str):
        self.where = model_dir
        single = os.path.join(model_dir, "model.safetensors")
        index = os.path.join(model_dir, "model.safetensors.index.json")
        self._files: List[SafetensorsFile] = []
        self._where_is: Dict[str, SafetensorsFile] = {}
        if os.path.exists(single):
            paths = [single]
        elif os.path.exists(index):
            with open(index, "r", encoding="utf-8") as f:
                try:
                    shard_of = json.load(f)["weight_map"]
                except (json.JSONDecodeError, KeyError, TypeError):
                    raise SafetensorsError(f"{index}: not a shard index (no 'weight_map')") from None
            paths = [os.path.join(model_dir, p) for p in sorted(set(shard_of.values()))]
        else:
            raise SafetensorsError(f"{model_dir}: neither model.safetensors nor model.safetensors.index.json found")
        for p in paths:
            sf = SafetensorsFile(p)
            self._files.append(sf)
            for name in sf.names():
                if name in self._where_is:
                    raise SafetensorsError(f"{p}: tensor '{name}' is also in {self._where_is[name].path}")
                self._where_is[name] = sf

    def names(self):
        return self._where_is.keys()

    def shape_dtype(self, name):
        e = self._where_is[name].entries[name]
        return e.shape, e.dtype

    def tensor(self, name):
        return self._where_is[name].tensor(name)


class MemorySource(TensorSource):
    where = "tensors in memory"

    def __init__(self, tensors: Dict[str, torch.Tensor]):
        self._t = tensors

    def names(self):
        return self._t.keys()

    def shape_dtype(self, name):
        t = self._t[name]
        return tuple(t.shape), t.dtype

    def tensor(self, name):
        return self._t[name]


def target_dtype(stored: torch.dtype, kind: str, engine_dtype: torch.dtype) -> torch.dtype:
    if kind == "int":
        return torch.int32
    if engine_dtype == torch.float32 or stored == torch.float32:
        return torch.float32
    return torch.bfloat16


def load_tensors(source: TensorSource, expected: Dict[str, TensorSpec], engine_dtype: torch.dtype,
                 device: torch.device, ignore: Iterable[str] = ()) -> Dict[str, torch.Tensor]:
    """Check ``source`` against ``expected`` (checkpoint name -> spec) and bring every expected
    tensor to ``device``.  ``ignore``: regular expressions of tensor names that may be present
    without being used."""
    have = set(source.names())
    ignore_re = [re.compile(p) for p in ignore]
    missing = sorted(n for n in expected if n not in have)
    unexpected = sorted(n for n in have if n not in expected and not any(r.fullmatch(n) for r in ignore_re))
    wrong = []
    for name, spec in expected.items():
        if name not in have:
            continue
        shape, dt = source.shape_dtype(name)
        if tuple(shape) != tuple(spec.shape):
            wrong.append(f"{name} is {list(shape)}, the configuration needs {list(spec.shape)}")
        elif spec.kind == "int" and dt.is_floating_point:
            wrong.append(f"{name} is {dt}, an integer table is needed")
        elif spec.kind == "float" and not dt.is_floating_point:
            wrong.append(f"{name} is {dt}, a float tensor is needed")
    if missing or unexpected or wrong:
        raise WeightError(source.where, missing, unexpected, wrong)
    out = {}
    for name, spec in expected.items():
        t = source.tensor(name)
        out[name] = t.to(device=device, dtype=target_dtype(t.dtype, spec.kind, engine_dtype)).contiguous()
    return out
