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


def run_part(role: str, kind: str, params: dict, tensors: dict, dtype="bfloat16", *, tokens=None, x=None, residual=None,
             out_cols: int = 0):
    """Build ONE part from its parameters and tensors, run it once on the GPU and return float32 numpy results
    (``fg_part_run``): norm: x [M, E] -> [M, E]; feed_forward: xn = x, returns residual + part(x); head: xn = x ->
    [M, out_cols]; embedding: tokens [M] -> [M, out_cols].  Mixers need a cache: ``Engine.block_forward``."""
    import json

    import numpy as np

    from ..weights import dtype_code, host_tensor_array
    arr, n, keep = host_tensor_array(tensors)
    tok_arr = None
    if tokens is not None:
        tok_arr, M = capi.int_array(tokens)
        cols_in = 0
    else:
        x = np.ascontiguousarray(x, dtype=np.float32)
        M, cols_in = x.shape
    res = np.ascontiguousarray(residual, dtype=np.float32).copy() if residual is not None else None
    cols_out = out_cols or cols_in
    out = np.zeros((M, cols_out), dtype=np.float32) if role != "feed_forward" else None
    capi.check(capi.lib().fg_part_run(ROLES[role], kind.encode("utf-8"), json.dumps(params).encode("utf-8"), dtype_code(dtype),
                                      arr, n, tok_arr, c_void_p(x.ctypes.data) if x is not None else None,
                                      c_void_p(res.ctypes.data) if res is not None else None,
                                      c_void_p(out.ctypes.data) if out is not None else None, M, cols_in, cols_out))
    return res if role == "feed_forward" else out


def position_tables(kind: str, params: dict, max_positions: int):
    """(cos, sin [max_positions, head_dim / 2], row permutation [head_dim]) of a position encoding."""
    import json

    import numpy as np
    hd = int(params["head_dim"])
    cos = np.zeros((max_positions, hd // 2), dtype=np.float32)
    sin = np.zeros_like(cos)
    perm = (ctypes.c_int * hd)()
    capi.check(capi.lib().fg_position_tables(kind.encode("utf-8"), json.dumps(params).encode("utf-8"), int(max_positions),
                                             c_void_p(cos.ctypes.data), c_void_p(sin.ctypes.data), perm))
    return cos, sin, list(perm)
