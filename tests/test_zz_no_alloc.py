"""fg_attention_decode_noalloc, the entry point for callers that cannot allocate device memory
(see fastgguf_b200/csrc/fastgguf_noalloc.h): called through its exported C symbol and compared
with the existing entry point fg_attention_decode on its scratch-memory path, on two calls in a
row (the fixed scratch array keeps the first call's contents when the second one runs).

This file sorts last, so a run that stops at the first failure has run every other test first.
"""
import ctypes
import math
from ctypes import c_float, c_int, c_void_p

import pytest
import torch

from test_kernels_attention import _err, make_case, plain

pytestmark = pytest.mark.gpu


def _noalloc_symbol():
    from fastgguf_b200.csrc.build import build_module
    lib = ctypes.CDLL(build_module("attn"))              # the plain C symbol, no framework wrapper
    fn = lib.fg_attention_decode_noalloc
    fn.restype = c_int
    fn.argtypes = [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                   c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p]
    return fn


def _call(fn, case, H, KV, hd, scale, n_splits):
    q = case["q"]
    out = torch.empty((q.shape[0], H * hd), dtype=torch.bfloat16, device="cuda")
    rc = fn(q.data_ptr(), q.stride(0), out.data_ptr(), out.stride(0), case["positions"].data_ptr(),
            case["table"].data_ptr(), case["table"].shape[1], case["k_pool"].data_ptr(), case["v_pool"].data_ptr(),
            q.shape[0], H, KV, hd, 64, scale, 0, n_splits, torch.cuda.current_stream().cuda_stream)
    return rc, out


@pytest.mark.parametrize("H,KV,hd", [(8, 2, 64), (6, 2, 128)])
def test_noalloc_matches_existing_entry_point_twice(H, KV, hd):
    from fastgguf_b200.ops import fast_attention
    fn = _noalloc_symbol()
    scale = 1.0 / math.sqrt(hd)
    # two different problems back to back: the second call finds the first one's partials in the array
    for seed, lens, n_splits in ((21, [0, 63, 700, 129], 5), (22, [300, 5, 1000], 3), (23, [17], 1)):
        case = make_case(lens, [1] * len(lens), H, KV, hd, torch.bfloat16, seed)
        want = fast_attention.attention_decode(case["q"], case["positions"], case["table"], case["k_pool"],
                                               case["v_pool"], H, KV, hd, scale, 0, n_splits=n_splits,
                                               use_scratch=True)
        rc, got = _call(fn, case, H, KV, hd, scale, n_splits)
        assert rc == 0
        torch.cuda.synchronize()
        assert torch.equal(got, want)                    # same kernels, same order of operations
        assert _err(got, plain(case, H, KV, hd, scale, 0)) < 1.5e-2


def test_noalloc_rejects_requests_beyond_its_array():
    fn = _noalloc_symbol()
    H, KV, hd = 32, 8, 128
    case = make_case([10] * 4, [1] * 4, H, KV, hd, torch.bfloat16, 24)
    case["q"] = case["q"].repeat(300, 1)                 # B * H * n_splits * (hd + 2) > 1 Mi floats
    rc, _ = _call(fn, dict(case), H, KV, hd, 0.1, 2)
    assert rc == 10005                                   # refused before anything is launched
    rc, _ = _call(fn, dict(case), H, 0, hd, 0.1, 2)
    assert rc == 10002                                   # no KV heads: a size error, not a division by zero
    torch.cuda.synchronize()
