"""The parts a decoder layer is put together from live in the C++ host (``csrc/host/parts.cpp``): norm
("rmsnorm"), position encoding ("rope"), mixer ("gqa_attention"), feed-forward ("swiglu"), block arrangement
("prenorm"), embedding ("embedding") and head ("lm_head"), each built from a kind name and parameters of the
model spec, chosen layer by layer.

A kind the library does not have is added from outside, without a change to any file of the library: a shared
library that fills an ``fg_part_vtable`` (``csrc/fastgguf_parts.h``: create / tensor declarations / load / cache
and state requests / forward on the engine's stream) and is registered under a role and a kind name.  From
Python::

    from fastgguf_b200.parts import register_part_library
    lib = register_part_library("libmy_parts.so", {("mixer", "my_mixer"): "my_mixer_vtable"})

where ``my_mixer_vtable`` is an exported function ``const fg_part_vtable *my_mixer_vtable(void)``.
"""
from __future__ import annotations

import ctypes
from ctypes import c_void_p
from typing import Dict, Tuple

from .. import capi

ROLES = dict(capi.ROLE)
_libraries = []


def register_part(role: str, kind: str, vtable_pointer) -> None:
    """Register the table of functions at ``vtable_pointer`` as the ``kind`` of ``role``."""
    if role not in ROLES:
        raise ValueError(f"unknown role '{role}' (known: {', '.join(ROLES)})")
    capi.check(capi.lib().fg_register_part(ROLES[role], kind.encode("utf-8"), c_void_p(vtable_pointer)))


def register_part_library(path: str, kinds: Dict[Tuple[str, str], str]) -> ctypes.CDLL:
    """Load a shared library and register ``kinds``: (role, kind name) -> name of the exported function that
    returns the kind's ``fg_part_vtable``."""
    lib = ctypes.CDLL(path)
    _libraries.append(lib)                       # the host keeps pointers into it
    for (role, kind), symbol in kinds.items():
        fn = getattr(lib, symbol)
        fn.restype, fn.argtypes = c_void_p, []
        register_part(role, kind, fn())
    return lib
