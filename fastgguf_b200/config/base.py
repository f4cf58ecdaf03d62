"""Typed model configuration: the shared base and the error type.

A configuration is read from the architecture's own ``config.json`` keys.  Every size and
every constant that ``config.json`` gives lives in the typed object and nowhere else; code
that needs a size takes it from there (or from a part's parameters, which were filled from
there).

The reference engine reads the same numbers from GGUF metadata through ``kv_num(g, key,
default)`` (fastgguf.c:448-454) with an architecture prefix (fastgguf.c:4189) and fails with
"bad config" on nonsense (fastgguf.c:4215-4218).
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, fields, asdict
from typing import ClassVar


class ConfigError(ValueError):
    """A config.json that is missing a key, has a wrong type, or describes an impossible model."""


_MISSING = object()


def take(d: dict, key: str, typ, default=_MISSING, *, where: str = "config.json"):
    """Fetch ``d[key]`` with a type check; ``default`` stands for an absent or null key."""
    v = d.get(key, None)
    if v is None:
        if default is _MISSING:
            raise ConfigError(f"{where}: required key '{key}' is missing")
        return default
    if typ is float and isinstance(v, int) and not isinstance(v, bool):
        v = float(v)
    if typ is int and isinstance(v, bool):
        raise ConfigError(f"{where}: key '{key}' must be an integer, got {v!r}")
    if typ is int and isinstance(v, float) and v == int(v):
        v = int(v)
    if not isinstance(v, typ):
        raise ConfigError(f"{where}: key '{key}' must be {typ.__name__}, got {type(v).__name__} ({v!r})")
    return v


@dataclass
class ModelConfig:
    """Base of every architecture's typed configuration."""

    #: names under which ``architectures[0]`` of config.json selects this class
    architecture_names: ClassVar[tuple] = ()

    @classmethod
    def from_dict(cls, d: dict) -> "ModelConfig":  # pragma: no cover - abstract
        raise NotImplementedError

    def to_dict(self) -> dict:
        """The config.json form of this configuration (what ``from_dict`` reads back)."""
        raise NotImplementedError

    def validate(self) -> None:
        raise NotImplementedError

    # -- shared helpers ---------------------------------------------------------------
    def describe(self) -> dict:
        """Every field, plus derived sizes; the ``inspect`` dump prints this."""
        out = {}
        for f in fields(self):
            v = getattr(self, f.name)
            out[f.name] = asdict(v) if hasattr(v, "__dataclass_fields__") else v
        return out


def read_config_json(model_dir: str) -> dict:
    path = os.path.join(model_dir, "config.json")
    try:
        with open(path, "r", encoding="utf-8") as f:
            d = json.load(f)
    except FileNotFoundError:
        raise ConfigError(f"{path}: no such file") from None
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path}: not valid JSON ({e})") from None
    if not isinstance(d, dict):
        raise ConfigError(f"{path}: top level must be an object")
    return d


def merge_generation_config(model_dir: str, d: dict) -> dict:
    """Stop tokens that a model folder names beside config.json: ``generation_config.json`` may list further
    ``eos_token_id`` values (instruction-tuned checkpoints end a turn with tokens that config.json does not name).
    The union, config.json's first, replaces ``d["eos_token_id"]``; a folder without the file is left as it is.
    (The reference takes its stop set from the model file's metadata plus named control tokens,
    fastgguf.c:3644-3652.)"""
    path = os.path.join(model_dir, "generation_config.json")
    if not os.path.exists(path):
        return d
    try:
        with open(path, "r", encoding="utf-8") as f:
            g = json.load(f)
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path}: not valid JSON ({e})") from None
    more = g.get("eos_token_id") if isinstance(g, dict) else None
    if more is None:
        return d
    more = [more] if isinstance(more, int) and not isinstance(more, bool) else more
    if not isinstance(more, list) or not all(isinstance(t, int) and not isinstance(t, bool) for t in more):
        raise ConfigError(f"{path}: 'eos_token_id' must be an integer or a list of integers, got {more!r}")
    have = d.get("eos_token_id")
    have = [] if have is None else [have] if isinstance(have, int) and not isinstance(have, bool) else have
    if not isinstance(have, list):
        return d                                     # config.json's own value is wrong: its reader says so
    merged = list(have) + [t for t in more if t not in have]
    out = dict(d)
    out["eos_token_id"] = merged[0] if len(merged) == 1 else merged
    return out


def architecture_name(d: dict) -> str:
    archs = d.get("architectures")
    if not isinstance(archs, list) or not archs or not isinstance(archs[0], str):
        raise ConfigError("config.json: 'architectures' must be a non-empty list of names")
    return archs[0]
