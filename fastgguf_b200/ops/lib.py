"""Loading the kernel libraries and calling their ``extern "C"`` launchers.

Every launcher takes raw device pointers, sizes and the CUDA stream, and returns 0 or an error
code.  The wrappers here pass ``tensor.data_ptr()`` and torch's current stream, so launches
take part in stream capture like any other kernel.  A missing library or a failed launch
raises: there is no other implementation to fall back to.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_void_p

import torch

from ..csrc.build import load_module

FG_F32, FG_BF16 = 0, 1

_ERRORS = {
    10001: "unsupported dtype combination",
    10002: "a size outside what this kernel takes",
    10003: "device-side wait ran out (pipeline error flag set)",
    10004: "could not encode a TMA tensor map",
    10005: "the request exceeds the fixed scratch array of the no-allocation entry point",
}


class KernelError(RuntimeError):
    pass


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.float32:
        return FG_F32
    if dt == torch.bfloat16:
        return FG_BF16
    raise KernelError(f"kernels take float32 and bfloat16 tensors, got {dt}")


def ptr(t) -> c_void_p:
    return c_void_p(0 if t is None else t.data_ptr())


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def stream() -> c_void_p:
    """The current CUDA stream of the current device, as a handle for the launchers.  Asked through the
    raw-stream call when this torch has it: ``torch.cuda.current_stream()`` builds a Stream object on every
    call (7 us), a third of the host time of a step launched kernel by kernel."""
    if _raw_stream is not None:
        return c_void_p(_raw_stream(torch.cuda.current_device()))
    return c_void_p(torch.cuda.current_stream().cuda_stream)


#: launcher calls made so far (each launches at least one kernel of this library)
launch_count = 0


def launches() -> int:
    return launch_count


def check(code: int, what: str) -> None:
    global launch_count
    launch_count += 1
    if code != 0:
        msg = _ERRORS.get(code)
        if msg is None:
            msg = f"CUDA error {code}"
        raise KernelError(f"{what}: {msg}")


def require_cuda(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("fastgguf_b200 kernels run on a CUDA device only; got a tensor on "
                              f"'{t.device}' (there is no CPU path)")


_SIGNATURES = {
    "core": {
        "fg_embed_gather": [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_void_p],
        "fg_embed_gather_norm": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                 c_void_p],
        "fg_rmsnorm": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p],
        "fg_rope_append": [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                           c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p],
        "fg_silu_mul": [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
        "fg_gemm_generic": [c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_int,
                            c_int, c_int, c_int, c_void_p],
        "fg_attention_generic": [c_void_p, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int,
                                 c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p],
        "fg_sample": [c_void_p, c_int, c_int, c_int, c_float, c_int, c_float, c_float, c_int, c_void_p,
                      c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p],
        "fg_argmax": [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p],
        "fg_decode_advance": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p],
    },
}

_libs: dict = {}


def register_signatures(module: str, signatures: dict) -> None:
    _SIGNATURES.setdefault(module, {}).update(signatures)


#: (library, reader of its device-side error flag): a bounded wait that ran out leaves wrong output behind
_ERROR_FLAGS = (("tc", "fg_gemm_tc_error"), ("attn", "fg_attention_prefill_tc_error"))


def raise_on_device_error(where: str = "") -> None:
    """Raise if a bounded wait inside a kernel ran out since the last call (the flags are cleared).

    Reads only the libraries that were loaded; the read synchronises, so callers use it where they
    wait for the device anyway (after a prompt step, at the end of a batch, before logits are written)."""
    for module, reader in _ERROR_FLAGS:
        l = _libs.get(module)
        if l is None:
            continue
        code = int(getattr(l, reader)())
        if code != 0:
            raise KernelError(f"{where or 'kernel'}: a device-side wait ran out in library '{module}' "
                              f"(code {code >> 8}, role {code & 255}); its output is not valid")


def lib(module: str = "core") -> ctypes.CDLL:
    l = _libs.get(module)
    if l is None:
        l = load_module(module)
        for name, argtypes in _SIGNATURES.get(module, {}).items():
            fn = getattr(l, name)
            fn.argtypes = argtypes
            fn.restype = c_int
        _libs[module] = l
    return l
