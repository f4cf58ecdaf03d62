"""Typed model configuration as Python sees it: a view of the C++ host's configuration object.

The configuration is read, defaulted and validated by the host (``csrc/host/config.cpp``: the
architecture's own config.json keys, the reference's defaults for absent ones - fastgguf.c:4224,
:4228, :4281-4283 - and "bad config" errors, :4215-4218).  A ``ModelConfig`` here holds the host's
handle and shows its fields as attributes; no size or constant of config.json is kept anywhere else.
"""
from __future__ import annotations

import json
import os
from ctypes import byref, c_void_p
from types import SimpleNamespace

from .. import capi
from ..capi import ConfigError

__all__ = ["ConfigError", "ModelConfig", "architecture_name", "read_config_json"]


class ModelConfig:
    """A configuration of a registered architecture (a handle of the host plus its description)."""

    def __init__(self, handle: c_void_p):
        self._handle = handle
        self._desc = capi.take_json(capi.lib().fg_config_describe, handle)

    def __del__(self):
        h, self._handle = getattr(self, "_handle", None), None
        if h:
            try:
                capi.lib().fg_config_destroy(h)
            except Exception:
                pass

    # -- construction ------------------------------------------------------------------
    @classmethod
    def from_dict(cls, d: dict) -> "ModelConfig":
        out = c_void_p()
        capi.check(capi.lib().fg_config_from_json(json.dumps(d).encode("utf-8"), byref(out)))
        return cls(out)

    @classmethod
    def from_dir(cls, model_dir: str) -> "ModelConfig":
        out = c_void_p()
        capi.check(capi.lib().fg_config_from_dir(os.fspath(model_dir).encode("utf-8"), byref(out)))
        return cls(out)

    # -- views ---------------------------------------------------------------------------
    @property
    def architecture(self) -> str:
        return self._desc["architecture"]

    @property
    def architecture_names(self) -> tuple:
        return (self._desc["architecture"],)

    def to_dict(self) -> dict:
        """The config.json form of this configuration (what ``from_dict`` reads back)."""
        return capi.take_json(capi.lib().fg_config_to_json, self._handle)

    def describe(self) -> dict:
        """Every field, plus derived sizes, memory per token and the keys that were defaulted."""
        return dict(self._desc)

    def spec_json(self) -> dict:
        """The model as data: parts, layers, execution order, checkpoint tensor names."""
        return capi.take_json(capi.lib().fg_config_spec, self._handle)

    def parameter_count(self) -> int:
        return int(self._desc["parameters"])

    def __getattr__(self, name):
        desc = self.__dict__.get("_desc")
        if desc is None or name not in desc:
            raise AttributeError(name)
        v = desc[name]
        if name == "eos_token_ids":
            return tuple(v)
        if isinstance(v, dict):
            return SimpleNamespace(**v)
        return v

    def __eq__(self, other):
        return isinstance(other, ModelConfig) and self.to_dict() == other.to_dict()

    __hash__ = None

    def __repr__(self):
        return f"{type(self).__name__}({self.to_dict()})"


def read_config_json(model_dir: str) -> dict:
    """config.json of a folder as it stands (for ``dump``); the typed reading is the host's."""
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


def architecture_name(d: dict) -> str:
    archs = d.get("architectures")
    if not isinstance(archs, list) or not archs or not isinstance(archs[0], str):
        raise ConfigError("config.json: 'architectures' must be a non-empty list of names")
    return archs[0]
