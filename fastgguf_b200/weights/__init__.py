"""Weights: what the C++ host does with them, reachable from Python.

The safetensors reader, the check of a checkpoint against what a model's parts declare (ONE error that lists
missing, unexpected and wrongly shaped tensors), the dtype policy and the seeded random-weights writer are the
host's (``csrc/host/safetensors.cpp``, ``csrc/host/model.cpp``); this module marshals.  dtype policy: in the
bfloat16 engine, float tensors stored in 16 bits become bfloat16, a tensor stored in 32 bits stays float32,
integer tables become int32; the float32 engine widens every float tensor.
"""
from __future__ import annotations

import json
import os
from typing import Dict, Optional

from .. import capi
from ..capi import SafetensorsError, WeightError

__all__ = ["WeightError", "SafetensorsError", "write_random_model", "folder_tensors", "expected_tensors",
           "check_weights", "host_tensor_array", "dtype_code"]

_DTYPE_CODES = {"float32": capi.FG_F32, "fp32": capi.FG_F32, "f32": capi.FG_F32, "bfloat16": capi.FG_BF16,
                "bf16": capi.FG_BF16}


def dtype_code(dtype) -> int:
    """FG_F32 / FG_BF16 from a name or a torch dtype."""
    name = str(dtype).replace("torch.", "").lower()
    try:
        return _DTYPE_CODES[name]
    except KeyError:
        raise ValueError(f"unknown dtype '{dtype}' (known: bfloat16, float32)") from None


def write_random_model(config, seed: int, out_dir: str, dtype="bfloat16") -> str:
    """Write ``out_dir/config.json`` and ``out_dir/model.safetensors`` from a configuration and a seed:
    weights ~ N(0, 0.02), norm weights 1 + N(0, 0.01); returns ``out_dir``."""
    os.makedirs(out_dir, exist_ok=True)
    capi.check(capi.lib().fg_write_random_model(config._handle, int(seed) & (2 ** 64 - 1), os.fspath(out_dir).encode("utf-8"),
                                                dtype_code(dtype)))
    return os.fspath(out_dir)


def folder_tensors(model_dir: str) -> list:
    """[{"name", "dtype", "shape"}] of a model folder, read by the host's safetensors reader."""
    return capi.take_json(capi.lib().fg_folder_tensors, os.fspath(model_dir).encode("utf-8"))


def _spec_text(config_or_spec) -> bytes:
    spec = config_or_spec.spec_json() if hasattr(config_or_spec, "spec_json") else config_or_spec
    if hasattr(spec, "to_json"):
        spec = spec.to_json()
    return json.dumps(spec).encode("utf-8")


def expected_tensors(config_or_spec) -> dict:
    """Checkpoint name -> {"shape", "kind", "init", "std"} of every tensor the model's parts declare."""
    return capi.take_json(capi.lib().fg_spec_tensors, _spec_text(config_or_spec))


_TORCH_CODES = None


def host_tensor_array(tensors: Dict[str, object]):
    """A ctypes array of fg_host_tensor for CPU tensors (torch or numpy); returns (array, keep_alive)."""
    global _TORCH_CODES
    import numpy as np
    keep, items = [], []
    for name, t in tensors.items():
        if hasattr(t, "detach"):                                  # a torch tensor
            import torch
            if _TORCH_CODES is None:
                _TORCH_CODES = {torch.float32: capi.FG_F32, torch.bfloat16: capi.FG_BF16, torch.float16: capi.FG_F16,
                                torch.int32: capi.FG_I32, torch.int64: capi.FG_I64}
            t = t.detach().cpu().contiguous()
            if t.dtype not in _TORCH_CODES:
                raise WeightError(f"tensor '{name}': unsupported type {t.dtype}")
            code, shape, ptr = _TORCH_CODES[t.dtype], tuple(t.shape), t.data_ptr()
        else:
            t = np.ascontiguousarray(t)
            codes = {"float32": capi.FG_F32, "float16": capi.FG_F16, "int32": capi.FG_I32, "int64": capi.FG_I64}
            if t.dtype.name not in codes:
                raise WeightError(f"tensor '{name}': unsupported type {t.dtype}")
            code, shape, ptr = codes[t.dtype.name], t.shape, t.ctypes.data
        if len(shape) > 4:
            raise WeightError(f"tensor '{name}' has {len(shape)} dimensions (at most 4)")
        keep.append(t)
        h = capi.HostTensor()
        h.name, h.dtype, h.ndim, h.data = name.encode("utf-8"), code, len(shape), ptr
        for i, s in enumerate(shape):
            h.shape[i] = int(s)
        items.append(h)
    arr = (capi.HostTensor * max(1, len(items)))(*items)
    return arr, len(items), keep


def check_weights(config_or_spec, model_dir: Optional[str] = None, tensors: Optional[dict] = None,
                  dtype="bfloat16") -> dict:
    """Check a folder (or tensors in memory) against the model without a device; raises ONE ``WeightError``
    listing everything that is wrong, else returns checkpoint name -> the dtype it takes in an engine of ``dtype``."""
    if model_dir is not None:
        return capi.take_json(capi.lib().fg_check_weights, _spec_text(config_or_spec), os.fspath(model_dir).encode("utf-8"),
                              None, 0, dtype_code(dtype))
    arr, n, keep = host_tensor_array(tensors or {})
    return capi.take_json(capi.lib().fg_check_weights, _spec_text(config_or_spec), None, arr, n, dtype_code(dtype))
