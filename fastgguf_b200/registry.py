"""One registry from an architecture's name to its model.

``architectures[0]`` of config.json selects an :class:`Architecture`: the typed configuration
class that reads the file and a function that turns the configuration into a
:class:`~fastgguf_b200.engine.spec.ModelSpec` (which parts, in which layers, run in which
order, with which checkpoint tensor names).  Everything else in the framework (loader, cache,
step function, generation, replay) works from the spec and never asks which model it is in.

The reference picks its code path by ``strcmp`` on ``general.architecture`` and carries on
with the Llama path for unknown names (fastgguf.c:4191-4198).  Here an unknown name is an
error that lists what is registered.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict

from .config.base import ConfigError, ModelConfig, architecture_name, merge_generation_config, read_config_json


@dataclass(frozen=True)
class Architecture:
    name: str
    config_class: type
    build_spec: Callable  # (config) -> ModelSpec


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(name: str, config_class: type, build_spec: Callable) -> None:
    _ARCHITECTURES[name] = Architecture(name, config_class, build_spec)


def registered_architectures() -> list:
    _load_builtin()
    return sorted(_ARCHITECTURES)


def get_architecture(name: str) -> Architecture:
    _load_builtin()
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        raise ConfigError(
            f"architecture '{name}' is not registered (registered: {', '.join(sorted(_ARCHITECTURES)) or 'none'})"
        ) from None


def config_from_dict(d: dict) -> ModelConfig:
    arch = get_architecture(architecture_name(d))
    return arch.config_class.from_dict(d)


def config_from_dir(model_dir: str) -> ModelConfig:
    return config_from_dict(merge_generation_config(model_dir, read_config_json(model_dir)))


def spec_from_config(config: ModelConfig):
    name = type(config).architecture_names[0]
    return get_architecture(name).build_spec(config)


_loaded = False


def _load_builtin() -> None:
    global _loaded
    if not _loaded:
        _loaded = True
        from .models import llama  # noqa: F401  (registers itself)
