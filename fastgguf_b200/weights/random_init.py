"""Random weights: a model folder (config.json, model.safetensors) from a configuration and a seed.

Reference counterpart: the fixture generator ``tools/synth_gguf.py`` - real shapes, seeded
random values, weights ~ N(0, 0.02) (tools/synth_gguf.py:50, :83-86), norm weights 1
(:166, :171; here 1 + N(0, 0.01) so that a forgotten norm weight shows).  Each tensor has its
own generator seeded from (seed, tensor name), so a tensor's values do not depend on which
other tensors exist or in which order they are drawn.
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Dict

import torch

from ..config.base import ModelConfig
from ..parts.base import Runtime, TensorSpec
from .safetensors_io import write_safetensors


def _tensor_seed(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(h[:8], "little") & 0x7FFFFFFFFFFFFFFF


def random_tensor(name: str, spec: TensorSpec, seed: int, dtype: torch.dtype, device="cpu") -> torch.Tensor:
    """One tensor's values.  The values depend on (seed, name) and on the kind of ``device`` (the CPU
    and CUDA generators differ); model folders are always written from the CPU generator."""
    g = torch.Generator(device=device)
    g.manual_seed(_tensor_seed(seed, name))
    if spec.kind == "int":
        return torch.zeros(spec.shape, dtype=torch.int32, device=device)
    kind, std = spec.init
    t = torch.randn(spec.shape, generator=g, dtype=torch.float32, device=device) * std
    if kind == "one_plus_normal":
        t = t + 1.0
    elif kind != "normal":
        raise ValueError(f"unknown initialisation '{kind}' for tensor {name}")
    return t.to(dtype)


def random_tensors(config: ModelConfig, seed: int, dtype: torch.dtype = torch.bfloat16,
                   device="cpu") -> Dict[str, torch.Tensor]:
    """Tensors by checkpoint name for ``config``, stored as ``dtype`` (on the CPU unless told otherwise)."""
    from ..engine.model import DecoderModel
    from ..registry import spec_from_config
    model = DecoderModel(spec_from_config(config), Runtime(torch.device("cpu"), dtype))
    return {name: random_tensor(name, spec, seed, dtype, device) for name, spec in model.expected_tensors().items()}


def write_random_model(config: ModelConfig, seed: int, out_dir: str, dtype: torch.dtype = torch.bfloat16) -> str:
    """Write ``out_dir/config.json`` and ``out_dir/model.safetensors``; returns ``out_dir``."""
    os.makedirs(out_dir, exist_ok=True)
    d = config.to_dict()
    d["torch_dtype"] = {torch.bfloat16: "bfloat16", torch.float32: "float32", torch.float16: "float16"}[dtype]
    with open(os.path.join(out_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(d, f, indent=2)
    write_safetensors(os.path.join(out_dir, "model.safetensors"), random_tensors(config, seed, dtype),
                      metadata={"format": "pt", "seed": str(seed)})
    return out_dir
