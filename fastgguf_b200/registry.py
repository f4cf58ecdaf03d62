"""One registry from an architecture's name to its model - the host's (``csrc/host/config.cpp``).

``architectures[0]`` of config.json selects the reader of the typed configuration and the function that
turns it into a model spec (which parts, in which layers, run in which order, with which checkpoint
tensor names).  Everything else (loader, cache, step function, generation, replay) works from the spec and
never asks which model it is in.  The reference picks its code path by ``strcmp`` on
``general.architecture`` and carries on with the Llama path for unknown names (fastgguf.c:4191-4198); here
an unknown name is an error that lists what is registered.
"""
from __future__ import annotations

import ctypes
import json
from typing import Callable

from . import capi
from .config.base import ModelConfig
from .config.llama import LlamaConfig
from .engine.spec import ModelSpec

_CLASSES = {"LlamaForCausalLM": LlamaConfig}
_keep_alive = []


def registered_architectures() -> list:
    return sorted(capi.take_json(capi.lib().fg_registered_architectures))


def register_architecture(name: str, build_spec: Callable[[dict], dict]) -> None:
    """Another architecture: ``build_spec(config_json_dict) -> model spec (dict)``; a raised exception refuses
    the configuration with its message."""
    libc = ctypes.CDLL(None)
    libc.malloc.restype, libc.malloc.argtypes = ctypes.c_void_p, [ctypes.c_size_t]

    def to_spec(config_json, err, err_cap, _user):
        try:
            text = json.dumps(build_spec(json.loads(config_json.decode("utf-8")))).encode("utf-8") + b"\0"
        except Exception as e:  # the message goes back to the host
            msg = str(e).encode("utf-8")[:max(0, err_cap - 1)]
            ctypes.memmove(err, msg + b"\0", len(msg) + 1)
            return None
        p = libc.malloc(len(text))
        ctypes.memmove(p, text, len(text))
        return p

    cb = capi.SPEC_BUILDER(to_spec)
    _keep_alive.append(cb)
    capi.check(capi.lib().fg_register_architecture(name.encode("utf-8"), cb, None))


def config_from_dict(d: dict) -> ModelConfig:
    archs = d.get("architectures") if isinstance(d, dict) else None
    cls = _CLASSES.get(archs[0], ModelConfig) if isinstance(archs, list) and archs else ModelConfig
    return ModelConfig.from_dict.__func__(cls, d)


def config_from_dir(model_dir: str) -> ModelConfig:
    cfg = ModelConfig.from_dir(model_dir)
    cfg.__class__ = _CLASSES.get(cfg.architecture, ModelConfig)
    return cfg


def spec_from_config(config: ModelConfig) -> ModelSpec:
    return ModelSpec.from_json(config.spec_json())
