"""bfloat16 tensor-core attention over the paged cache: a decode kernel (one new token per
sequence, pages split over CTAs; its fused form also rotates q and k and appends k and v), a
tcgen05 prefill kernel (128-row tiles of new tokens x query heads) and an mma.sync prefill kernel for
short pieces.  All take head sizes 64 and 128 and pages of 64 positions; ``supported`` says so, and the
caller uses the any-size kernel otherwise."""
from __future__ import annotations

from ctypes import c_float, c_int, c_void_p
from typing import Optional

import torch

from .lib import check, lib, ptr, register_signatures, stream

register_signatures("attn", {
    "fg_attention_decode": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                            c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p, c_void_p, c_void_p],
    "fg_attention_decode_fused": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                                  c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p],
    "fg_attention_prefill_tc": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                                c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p],
    "fg_attention_prefill_tc_error": [],
    "fg_attention_prefill_tc_variant": [c_int],
    "fg_attention_prefill": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                             c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p],
})

_n_sm = {}


def n_sm(device=None) -> int:
    """Streaming multiprocessors of the device (148 on a B200)."""
    idx = torch.cuda.current_device() if device is None else torch.device(device).index or 0
    if idx not in _n_sm:
        _n_sm[idx] = torch.cuda.get_device_properties(idx).multi_processor_count
    return _n_sm[idx]


def supported(q: torch.Tensor, k_pool: torch.Tensor, head_dim: int) -> bool:
    return (q.dtype == torch.bfloat16 and k_pool.dtype == torch.bfloat16 and head_dim in (64, 128)
            and k_pool.shape[2] == 64 and q.stride(1) == 1 and q.stride(0) % 2 == 0 and q.data_ptr() % 4 == 0)


def decode_splits(n_seq: int, n_heads: int, n_kv_heads: int, table_width: int, head_dim: int = 64) -> int:
    """How many CTAs share one sequence's pages: about one and a half CTAs per SM in all, and never more than fit
    on the GPU at once - three per SM at head size 64, one at 128 (each warp holds a K and a V page in shared
    memory), fewer beside the contraction kernels that are already resident.  What does not fit runs as a second
    wave whose page loads start late; measured at batch 8 with 8 KV heads and head size 64, 4 splits (256 CTAs)
    beat both 2 and 8, and at head size 128 two splits (128 CTAs) beat four.  Up to 8 splits (a power of two) are
    merged inside a thread-block cluster; only contexts beyond 16K positions take more splits and the
    scratch-memory path."""
    ctas = n_seq * n_kv_heads * ((n_heads // n_kv_heads + 15) // 16)
    if head_dim <= 64:
        want = (3 * n_sm() // 2 + ctas - 1) // ctas
    else:
        want = n_sm() // ctas
    want = max(1, min(want, table_width))
    if want > 8 and table_width > 256:
        return want
    s = 1
    while s < want and s < 8:
        s *= 2
    return s


def attention_decode(q, positions, block_table, k_pool, v_pool, n_heads, n_kv_heads, head_dim, scale, window=0,
                     n_splits: Optional[int] = None, out=None, use_scratch: bool = False):
    """q: [B, >= H*hd] bf16, one new token per sequence at ``positions[b]`` (already in the cache)."""
    B = q.shape[0]
    if n_splits is None:
        n_splits = decode_splits(B, n_heads, n_kv_heads, block_table.shape[1], head_dim)
    if out is None:
        out = torch.empty((B, n_heads * head_dim), dtype=torch.bfloat16, device=q.device)
    part_o = part_ml = None
    if n_splits not in (1, 2, 4, 8) or use_scratch:
        part_o = torch.empty((B, n_heads, n_splits, head_dim), dtype=torch.float32, device=q.device)
        part_ml = torch.empty((B, n_heads, n_splits, 2), dtype=torch.float32, device=q.device)
    check(lib("attn").fg_attention_decode(ptr(q), q.stride(0), ptr(out), out.stride(0), ptr(positions), ptr(block_table),
                                          block_table.shape[1], ptr(k_pool), ptr(v_pool), B, n_heads, n_kv_heads,
                                          head_dim, k_pool.shape[2], float(scale), int(window), n_splits,
                                          ptr(part_o), ptr(part_ml), stream()), "attention_decode")
    return out


def attention_prefill(q, cu_rows, seq_start, block_table, k_pool, v_pool, n_seq, max_new, n_heads, n_kv_heads,
                      head_dim, scale, window=0, out=None):
    """q: [rows, >= H*hd] bf16, sequences one after another; every new key/value is in the cache."""
    if out is None:
        out = torch.empty((q.shape[0], n_heads * head_dim), dtype=torch.bfloat16, device=q.device)
    check(lib("attn").fg_attention_prefill(ptr(q), q.stride(0), ptr(out), out.stride(0), ptr(cu_rows), ptr(seq_start),
                                           ptr(block_table), block_table.shape[1], ptr(k_pool), ptr(v_pool), n_seq,
                                           max_new, n_heads, n_kv_heads, head_dim, k_pool.shape[2], float(scale),
                                           int(window), stream()), "attention_prefill")
    return out


def attention_prefill_tc(q, cu_rows, seq_start, block_table, k_pool, v_pool, n_seq, max_new, n_heads, n_kv_heads,
                         head_dim, scale, window=0, out=None):
    """The same contract as ``attention_prefill`` on the tcgen05 tensor cores (128-row tiles, K/V by TMA,
    accumulators in tensor memory).  Needs 16-byte aligned rows of ``q`` and ``out``."""
    if out is None:
        out = torch.empty((q.shape[0], n_heads * head_dim), dtype=torch.bfloat16, device=q.device)
    check(lib("attn").fg_attention_prefill_tc(ptr(q), q.stride(0), ptr(out), out.stride(0), ptr(cu_rows), ptr(seq_start),
                                              ptr(block_table), block_table.shape[1], ptr(k_pool), ptr(v_pool),
                                              k_pool.shape[0], n_seq, max_new, n_heads, n_kv_heads, head_dim,
                                              k_pool.shape[2], float(scale), int(window), stream()),
          "attention_prefill_tc")
    return out


def prefill_tc_variant(bits: int) -> None:
    """Which form of the tcgen05 prefill attention runs: bit 0 / bit 1 = two score tiles in tensor memory at head
    size 64 / 128, bit 2 = with them at head size 64 two sets of softmax warps that take the iterations in turn;
    negative = chosen by head size and step shape (the default)."""
    check(lib("attn").fg_attention_prefill_tc_variant(int(bits)), "attention_prefill_tc_variant")


def prefill_tc_error() -> int:
    """0, or the code of the first bounded wait of the tcgen05 attention that ran out (clears it)."""
    return int(lib("attn").fg_attention_prefill_tc_error())


def attention_decode_fused(qkv, positions, block_table, k_pool, v_pool, cos, sin, n_heads, n_kv_heads, head_dim,
                           scale, window=0, n_splits: Optional[int] = None, out=None):
    """RoPE of q and of the new k, cache append and attention of one new token per sequence in ONE kernel.
    qkv: [B, >= (H + 2 KV) * hd] bf16 straight from the projection.  None when the step needs more than 8 splits
    (very long contexts): the caller then runs RoPE + append and attention separately."""
    B = qkv.shape[0]
    if n_splits is None:
        n_splits = decode_splits(B, n_heads, n_kv_heads, block_table.shape[1], head_dim)
    if n_splits not in (1, 2, 4, 8):
        return None
    if out is None:
        out = torch.empty((B, n_heads * head_dim), dtype=torch.bfloat16, device=qkv.device)
    check(lib("attn").fg_attention_decode_fused(ptr(qkv), qkv.stride(0), ptr(out), out.stride(0), ptr(positions),
                                                ptr(block_table), block_table.shape[1], ptr(k_pool), ptr(v_pool),
                                                ptr(cos), ptr(sin), B, n_heads, n_kv_heads, head_dim, k_pool.shape[2],
                                                float(scale), int(window), n_splits, stream()),
          "attention_decode_fused")
    return out
