"""ctypes bindings of the engine's C interface (``csrc/fastgguf_engine.h``, ``csrc/fastgguf_parts.h``).

The host of this framework is C++ (``csrc/host/``): configuration, weights, cache, the step function, the
generation loop and CUDA-graph handling live in ``libfg_engine.so``.  Everything in this Python package is
marshalling on top of it; this module loads the library, declares the argument types of its functions and
turns status codes into Python exceptions with the library's own message.
"""
from __future__ import annotations

import ctypes
import json
from ctypes import (CFUNCTYPE, POINTER, Structure, byref, c_char, c_char_p, c_float, c_int, c_int64, c_size_t,
                    c_uint64, c_void_p)

FG_F32, FG_BF16, FG_F16, FG_I32, FG_I64 = 0, 1, 2, 3, 4
ROLE = {"norm": 0, "position": 1, "mixer": 2, "feed_forward": 3, "block": 4, "embedding": 5, "head": 6}

OK, E_USAGE, E_CONFIG, E_WEIGHTS, E_CACHE, E_CAPACITY, E_TOKEN, E_DEVICE, E_KERNEL, E_INTERNAL = range(10)


class EngineError(RuntimeError):
    """A failed call of the C interface; ``code`` is its FG_E_* status."""

    code = E_INTERNAL

    def __init__(self, message: str, code: int = None):
        super().__init__(message)
        if code is not None:
            self.code = code


class UsageError(EngineError, ValueError):
    code = E_USAGE


class ConfigError(EngineError, ValueError):
    """A config.json that is missing a key, has a wrong type, or describes an impossible model."""
    code = E_CONFIG


class WeightError(EngineError, ValueError):
    """Missing, unexpected or wrongly shaped tensors (the message lists all of them), or a broken safetensors file."""
    code = E_WEIGHTS

    @staticmethod
    def _listed(message: str, label: str, sep: str):
        for line in message.splitlines():
            line = line.strip()
            if line.startswith(label):
                return [p for p in line.split(": ", 1)[1].split(sep)]
        return []

    @property
    def missing(self):
        return self._listed(str(self), "missing tensors", ", ")

    @property
    def unexpected(self):
        return self._listed(str(self), "unexpected tensors", ", ")

    @property
    def wrong(self):
        return self._listed(str(self), "wrong shapes or types", "; ")


SafetensorsError = WeightError


class CacheError(EngineError):
    code = E_CACHE


class CacheFull(CacheError):
    """No free slot, or not enough free pages for the tokens a step brings."""
    code = E_CAPACITY


class TokenError(EngineError, ValueError):
    code = E_TOKEN


class DeviceError(EngineError):
    code = E_DEVICE


class KernelError(EngineError):
    code = E_KERNEL


_BY_CODE = {E_USAGE: UsageError, E_CONFIG: ConfigError, E_WEIGHTS: WeightError, E_CACHE: CacheError,
            E_CAPACITY: CacheFull, E_TOKEN: TokenError, E_DEVICE: DeviceError, E_KERNEL: KernelError}


class HostTensor(Structure):
    _fields_ = [("name", c_char_p), ("dtype", c_int), ("ndim", c_int), ("shape", c_int64 * 4), ("data", c_void_p)]


class EngineOptions(Structure):
    _fields_ = [("dtype", c_int), ("max_batch", c_int), ("max_tokens", c_int64), ("max_seq_len", c_int),
                ("device", c_int), ("use_graphs", c_int), ("verbose", c_int), ("stream", c_void_p)]


class Sampling(Structure):
    _fields_ = [("temp", c_float), ("top_k", c_int), ("top_p", c_float), ("repeat_penalty", c_float),
                ("repeat_last_n", c_int), ("seed", c_uint64)]


TOKEN_CALLBACK = CFUNCTYPE(None, c_void_p, c_int, c_int)
ACQUIRE_FN = CFUNCTYPE(c_int, c_void_p, c_int, POINTER(c_int), c_int, POINTER(c_int))
RELEASE_FN = CFUNCTYPE(c_int, c_void_p, c_int)
STEP_FN = CFUNCTYPE(c_int, c_void_p, c_int, POINTER(c_int), POINTER(c_int), POINTER(c_int))
SAMPLE_FN = CFUNCTYPE(c_int, c_void_p, c_int, POINTER(c_int), POINTER(c_int))
ROOM_FN = CFUNCTYPE(c_int, c_void_p, c_int, POINTER(c_int))
BEGIN_FN = CFUNCTYPE(c_int, c_void_p, c_int, POINTER(c_int))
ADVANCE_FN = CFUNCTYPE(c_int, c_void_p, c_int, POINTER(c_int), POINTER(c_int))
CLOSE_FN = CFUNCTYPE(c_int, c_void_p)
SPEC_BUILDER = CFUNCTYPE(c_void_p, c_char_p, POINTER(c_char), c_size_t, c_void_p)


class LoopBackend(Structure):
    _fields_ = [("user", c_void_p), ("acquire", ACQUIRE_FN), ("release", RELEASE_FN), ("step", STEP_FN),
                ("sample", SAMPLE_FN), ("room", ROOM_FN)]


class LateBackend(Structure):
    _fields_ = [("user", c_void_p), ("begin", BEGIN_FN), ("advance", ADVANCE_FN), ("close", CLOSE_FN)]


P = POINTER
_SIGNATURES = {
    "fg_config_from_json": [c_char_p, P(c_void_p)],
    "fg_config_from_dir": [c_char_p, P(c_void_p)],
    "fg_config_to_json": [c_void_p, P(c_void_p)],
    "fg_config_describe": [c_void_p, P(c_void_p)],
    "fg_config_spec": [c_void_p, P(c_void_p)],
    "fg_registered_architectures": [P(c_void_p)],
    "fg_register_architecture": [c_char_p, SPEC_BUILDER, c_void_p],
    "fg_register_part": [c_int, c_char_p, c_void_p],
    "fg_write_random_model": [c_void_p, c_uint64, c_char_p, c_int],
    "fg_spec_tensors": [c_char_p, P(c_void_p)],
    "fg_folder_tensors": [c_char_p, P(c_void_p)],
    "fg_check_weights": [c_char_p, c_char_p, P(HostTensor), c_int, c_int, P(c_void_p)],
    "fg_engine_create": [c_void_p, c_char_p, P(EngineOptions), P(c_void_p)],
    "fg_engine_create_from_tensors": [c_void_p, P(HostTensor), c_int, P(EngineOptions), P(c_void_p)],
    "fg_engine_create_random": [c_void_p, c_uint64, P(EngineOptions), P(c_void_p)],
    "fg_engine_create_from_spec": [c_char_p, P(HostTensor), c_int, P(EngineOptions), P(c_void_p)],
    "fg_engine_info": [c_void_p, P(c_void_p)],
    "fg_engine_expected_tensors": [c_void_p, P(c_void_p)],
    "fg_slot_acquire": [c_void_p, P(c_int)],
    "fg_slot_release": [c_void_p, c_int],
    "fg_slot_length": [c_void_p, c_int, P(c_int)],
    "fg_engine_cache_check": [c_void_p],
    "fg_engine_free_pages": [c_void_p, c_int, P(c_int)],
    "fg_step": [c_void_p, c_int, P(c_int), P(c_int), P(c_int), c_int, P(c_int), c_void_p],
    "fg_engine_check_device": [c_void_p],
    "fg_engine_sampler_begin": [c_void_p, P(Sampling), P(c_int), c_int, c_int, c_uint64, P(c_int), c_int],
    "fg_engine_sample": [c_void_p, P(Sampling), P(c_int), c_int, c_void_p, c_int, P(c_int), P(c_int)],
    "fg_generate": [c_void_p, c_int, P(c_int), P(c_int64), P(Sampling), c_int, P(c_int), c_int, c_int, c_int,
                    TOKEN_CALLBACK, c_void_p, P(c_void_p)],
    "fg_result_get": [c_void_p, c_int, P(P(c_int)), P(c_int), P(c_int)],
    "fg_engine_stats": [c_void_p, P(c_void_p)],
    "fg_engine_profile": [c_void_p, c_int],
    "fg_engine_profile_report": [c_void_p, P(c_void_p)],
    "fg_session_begin": [c_void_p, c_int, P(c_int), P(c_int64), P(Sampling), P(c_int), c_int, P(c_void_p)],
    "fg_session_advance": [c_void_p, P(c_int), c_int],
    "fg_session_slots": [c_void_p, P(c_int)],
    "fg_run_batch": [P(LoopBackend), c_int, P(c_int), P(c_int64), c_int, c_int, P(c_int), c_int, TOKEN_CALLBACK,
                     c_void_p, P(c_void_p)],
    "fg_run_batch_late": [P(LateBackend), c_int, P(c_int), P(c_int64), c_int, c_int, P(c_int), c_int, c_int,
                          TOKEN_CALLBACK, c_void_p, P(c_void_p)],
    "fg_plan_batches": [c_int, c_int, P(c_void_p)],
    "fg_seed_resolve": [c_uint64, P(c_uint64)],
    "fg_seed_of_request": [c_uint64, c_uint64, P(c_uint64)],
    "fg_cache_create": [c_char_p, c_int64, c_int, c_int, c_int, P(c_void_p)],
    "fg_cache_acquire": [c_void_p, P(c_int)],
    "fg_cache_release": [c_void_p, c_int],
    "fg_cache_length": [c_void_p, c_int, P(c_int)],
    "fg_cache_reserve": [c_void_p, c_int, P(c_int), P(c_int)],
    "fg_cache_commit": [c_void_p, c_int, P(c_int), P(c_int)],
    "fg_cache_pages_needed": [c_void_p, c_int, c_int, P(c_int)],
    "fg_cache_free_pages": [c_void_p, c_int, P(c_int)],
    "fg_cache_block_table": [c_void_p, c_int, c_int, c_int, P(c_int)],
    "fg_cache_check": [c_void_p],
    "fg_cache_info": [c_void_p, P(c_void_p)],
    "fg_cache_bytes": [c_char_p, c_int64, c_int, c_int, P(c_void_p)],
    "fg_part_run": [c_int, c_char_p, c_char_p, c_int, P(HostTensor), c_int, P(c_int), c_void_p, c_void_p, c_void_p,
                    c_int, c_int, c_int],
    "fg_position_tables": [c_char_p, c_char_p, c_int, c_void_p, c_void_p, P(c_int)],
    "fg_engine_block_forward": [c_void_p, c_int, c_int, P(c_int), P(c_int), c_void_p],
}
_VOID = {"fg_config_destroy": [c_void_p], "fg_engine_destroy": [c_void_p], "fg_result_destroy": [c_void_p],
         "fg_cache_destroy": [c_void_p], "fg_session_close": [c_void_p], "fg_free": [c_void_p],
         "fg_engine_default_options": [P(EngineOptions)], "fg_sampling_default": [P(Sampling)]}

_lib = None


def lib() -> ctypes.CDLL:
    """libfg_engine.so, built on first use (no GPU is needed to build or to load it)."""
    global _lib
    if _lib is None:
        from .csrc.build import load_module
        l = load_module("engine")
        for name, args in _SIGNATURES.items():
            fn = getattr(l, name)
            fn.argtypes, fn.restype = args, c_int
        for name, args in _VOID.items():
            fn = getattr(l, name)
            fn.argtypes, fn.restype = args, None
        l.fg_last_error.argtypes, l.fg_last_error.restype = [], c_char_p
        l.fg_result_count.argtypes, l.fg_result_count.restype = [c_void_p], c_int
        l.fg_engine_stream.argtypes, l.fg_engine_stream.restype = [c_void_p], c_void_p
        l.fg_session_launches_per_step.argtypes, l.fg_session_launches_per_step.restype = [c_void_p], c_int
        _lib = l
    return _lib


def check(code: int) -> None:
    if code != OK:
        msg = (lib().fg_last_error() or b"").decode("utf-8", "replace")
        raise _BY_CODE.get(code, EngineError)(msg, code)


def take_json(fn, *args):
    """Call ``fn(*args, &text)`` and parse the JSON text it hands out."""
    out = c_void_p()
    check(fn(*args, byref(out)))
    try:
        return json.loads(ctypes.string_at(out.value).decode("utf-8"))
    finally:
        lib().fg_free(out)


def int_array(values):
    values = [int(v) for v in values]
    return (c_int * max(1, len(values)))(*values), len(values)


def prompts_arrays(prompts):
    flat = [int(t) for p in prompts for t in p]
    offs = [0]
    for p in prompts:
        offs.append(offs[-1] + len(p))
    return (c_int * max(1, len(flat)))(*flat), (c_int64 * len(offs))(*offs)


def ensure_kernel_libraries(dtype_code: int) -> None:
    """Build (if stale) the kernel libraries an engine of this dtype opens by name."""
    from .csrc.build import build_module
    for module in (("core", "tc", "attn") if dtype_code == FG_BF16 else ("core",)):
        build_module(module)
