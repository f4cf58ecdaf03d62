"""The bounded waits of the tensor-core kernels, run once for real: a test hook makes the producer of a pipeline leave
its first stage incomplete (a copy is never issued, so a barrier never fires - nothing faults, traps or spins without
end) and shortens the wait limit to about a millisecond.  The kernel must give up, raise its error flag, free its tensor
memory and return; the NEXT ordinary launch must be correct, which it could not be with tensor memory still held."""
import math
import time
from ctypes import c_int, c_longlong

import pytest
import torch

pytestmark = pytest.mark.gpu

LIMIT = 2_000_000          # SM cycles: about a millisecond


def _hook(lib, name):
    fn = getattr(lib, name)
    fn.argtypes, fn.restype = [c_longlong, c_int], c_int
    return fn


def test_decode_contraction_gives_up_and_the_next_launch_is_correct():
    from fastgguf_b200 import ops
    from fastgguf_b200.ops import fast_gemm
    g = torch.Generator().manual_seed(3)
    a = torch.randn(8, 512, generator=g).bfloat16().cuda()
    w = torch.randn(128, 512, generator=g).bfloat16().cuda()
    want = fast_gemm.gemm_tc(a, w, out_dtype=torch.float32, force_splits=1)        # one CTA, no cluster
    torch.cuda.synchronize()
    assert fast_gemm.pipeline_error() == 0
    assert (want.double().cpu() - a.double().cpu() @ w.double().cpu().T).abs().max() < 1e-2 * want.abs().max().item()
    hook = _hook(ops.lib("tc"), "fg_gemm_tc_test_hook")
    try:
        assert hook(LIMIT, 1) == 0
        t0 = time.time()
        fast_gemm.gemm_tc(a, w, out_dtype=torch.float32, force_splits=1)           # its first stage never completes
        torch.cuda.synchronize()                                                   # ... and it returns all the same
        assert time.time() - t0 < 2.0
        code = fast_gemm.pipeline_error()
        assert code >> 8 == 10003 and (code & 255) in (1, 2, 3)                    # FG_ERR_PIPELINE, raised by a role
    finally:
        assert hook(0, 0) == 0
    assert fast_gemm.pipeline_error() == 0                                         # reading cleared the flag
    again = fast_gemm.gemm_tc(a, w, out_dtype=torch.float32, force_splits=1)
    torch.cuda.synchronize()
    assert fast_gemm.pipeline_error() == 0 and torch.equal(again, want)


@pytest.mark.parametrize("variant", [1, 5], ids=["two-score-tiles", "two-score-tiles-two-softmax-sets"])
def test_prefill_attention_gives_up_and_the_next_launch_is_correct(variant):
    """(In the form with two sets of softmax warps each row's two threads meet at a barrier after their loops: every
    thread gets there, whichever of its waits ran out.)"""
    from fastgguf_b200 import ops
    from fastgguf_b200.ops import fast_attention
    from test_kernels_attention import _err, make_case, plain
    fast_attention.prefill_tc_variant(variant)
    try:
        _attention_gives_up(ops, fast_attention, _err, make_case, plain)
    finally:
        fast_attention.prefill_tc_variant(-1)


def _attention_gives_up(ops, fast_attention, _err, make_case, plain):
    H, KV, hd = 4, 2, 64
    new = [130]
    case = make_case([70], new, H, KV, hd, torch.bfloat16, 31)
    scale = 1.0 / math.sqrt(hd)

    def run():
        out = fast_attention.attention_prefill_tc(case["q"], case["cu_rows"], case["seq_start"], case["table"], case["k_pool"],
                                                  case["v_pool"], 1, 130, H, KV, hd, scale, 0)
        torch.cuda.synchronize()
        return out

    want = run()
    assert fast_attention.prefill_tc_error() == 0 and _err(want, plain(case, H, KV, hd, scale, 0)) < 1.5e-2
    hook = _hook(ops.lib("attn"), "fg_attention_prefill_tc_test_hook")
    try:
        assert hook(LIMIT, 1) == 0
        t0 = time.time()
        run()
        assert time.time() - t0 < 2.0
        code = fast_attention.prefill_tc_error()
        assert code >> 8 == 10003
    finally:
        assert hook(0, 0) == 0
    assert fast_attention.prefill_tc_error() == 0
    again = run()
    assert fast_attention.prefill_tc_error() == 0 and torch.equal(again, want)
