"""One Python function per kernel.  Each checks shapes and dtypes, then launches on the current
stream.  None of them has a CPU or library fallback."""
from __future__ import annotations

from typing import Optional

import torch

from .lib import KernelError, check, dtype_code, lib, ptr, raise_on_device_error, require_cuda, stream

__all__ = [
    "KernelError", "raise_on_device_error", "embed_gather", "embed_gather_norm", "rmsnorm", "rope_append", "silu_mul", "gemm_generic",
    "attention_generic", "attention", "rope_attention", "sample", "argmax", "decode_advance",
]


def _i32(t: torch.Tensor, name: str) -> torch.Tensor:
    if t.dtype != torch.int32 or not t.is_contiguous():
        raise KernelError(f"{name} must be a contiguous int32 tensor, got {t.dtype}")
    return t


def embed_gather(table: torch.Tensor, tokens: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x[m, :] = table[tokens[m], :] as f32.  table: [V, E] f32 or bf16; tokens: [M] int32."""
    require_cuda(table, tokens)
    _i32(tokens, "tokens")
    V, E = table.shape
    M = tokens.numel()
    if out is None:
        out = torch.empty((M, E), dtype=torch.float32, device=table.device)
    if not table.is_contiguous() or out.shape != (M, E) or out.dtype != torch.float32:
        raise KernelError("embed_gather: table must be contiguous and out [M, E] f32")
    check(lib().fg_embed_gather(ptr(table), dtype_code(table.dtype), ptr(tokens), ptr(out), M, E, stream()),
          "embed_gather")
    return out


def embed_gather_norm(table: torch.Tensor, tokens: torch.Tensor, norm_weight: torch.Tensor, eps: float):
    """``embed_gather`` that also starts the first RMSNorm: returns (x, DeferredNorm)."""
    from .fast_gemm import DeferredNorm
    require_cuda(table, tokens, norm_weight)
    _i32(tokens, "tokens")
    V, E = table.shape
    M = tokens.numel()
    if norm_weight.dtype != torch.float32 or norm_weight.numel() != E or not table.is_contiguous():
        raise KernelError("embed_gather_norm: the norm weight must be float32 [E] and the table contiguous")
    x = torch.empty((M, E), dtype=torch.float32, device=table.device)
    xw = torch.empty((M, E), dtype=torch.bfloat16, device=table.device)
    ss = torch.empty((1, M), dtype=torch.float32, device=table.device)
    check(lib().fg_embed_gather_norm(ptr(table), dtype_code(table.dtype), ptr(tokens), ptr(x), ptr(norm_weight),
                                     ptr(xw), ptr(ss), M, E, stream()), "embed_gather_norm")
    return x, DeferredNorm(xw, ss, 1, E, float(eps), x, norm_weight)


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out_dtype: torch.dtype,
            rows: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[r] = x[rows[r]] * rsqrt(mean(x^2) + eps) * weight.  x: [M, E] f32; weight: [E] f32."""
    require_cuda(x, weight, rows)
    if x.dtype != torch.float32 or weight.dtype != torch.float32 or not x.is_contiguous():
        raise KernelError("rmsnorm: x and weight must be float32 (the residual stream and the statistics are 32-bit)")
    M, E = x.shape
    if weight.numel() != E:
        raise KernelError(f"rmsnorm: weight has {weight.numel()} elements, rows have {E}")
    R = M if rows is None else _i32(rows, "rows").numel()
    if out is None:
        out = torch.empty((R, E), dtype=out_dtype, device=x.device)
    check(lib().fg_rmsnorm(ptr(x), ptr(weight), ptr(rows), ptr(out), dtype_code(out.dtype), R, E, float(eps),
                           stream()), "rmsnorm")
    return out


def rope_append(qkv: torch.Tensor, positions: torch.Tensor, row_seq: torch.Tensor,
                block_table: torch.Tensor, k_pool: Optional[torch.Tensor], v_pool: Optional[torch.Tensor],
                cos: torch.Tensor, sin: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int,
                write_kv: bool = True) -> None:
    """Rotate q (and k) of every row at the row's position; write k, v into the paged cache.

    qkv: [M, H*hd (+ 2*KV*hd)]; pools: [n_pages, KV, page, hd]; cos, sin: [max_pos, hd/2] f32.
    """
    require_cuda(qkv, positions, row_seq, block_table, cos, sin)
    M, ld = qkv.shape
    need = n_heads * head_dim + (2 * n_kv_heads * head_dim if write_kv else 0)
    if ld < need or not qkv.is_contiguous():
        raise KernelError(f"rope_append: rows of {ld} elements cannot hold {need}")
    if cos.shape[1] * 2 != head_dim or cos.dtype != torch.float32 or sin.shape != cos.shape:
        raise KernelError("rope_append: cos/sin tables must be [max_pos, head_dim/2] float32")
    page_size = 1
    if write_kv:
        if k_pool is None or v_pool is None or k_pool.dtype != qkv.dtype or v_pool.dtype != qkv.dtype:
            raise KernelError("rope_append: cache pools must have the dtype of qkv")
        if tuple(k_pool.shape[1:]) != (n_kv_heads, k_pool.shape[2], head_dim) or k_pool.shape != v_pool.shape:
            raise KernelError(f"rope_append: pools must be [pages, {n_kv_heads}, page, {head_dim}], got {tuple(k_pool.shape)}")
        page_size = k_pool.shape[2]
    check(lib().fg_rope_append(ptr(qkv), dtype_code(qkv.dtype), ld, ptr(_i32(positions, "positions")),
                               ptr(_i32(row_seq, "row_seq")), ptr(_i32(block_table, "block_table")),
                               block_table.shape[-1], ptr(k_pool), ptr(v_pool), ptr(cos), ptr(sin),
                               M, n_heads, n_kv_heads, head_dim, page_size, int(write_kv), stream()),
          "rope_append")


def silu_mul(gate_up: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[m, f] = silu(gate_up[m, f]) * gate_up[m, F + f]."""
    require_cuda(gate_up)
    M, F2 = gate_up.shape
    F = F2 // 2
    if F2 % 2 or not gate_up.is_contiguous():
        raise KernelError("silu_mul: input must be contiguous [M, 2F]")
    if out is None:
        out = torch.empty((M, F), dtype=gate_up.dtype, device=gate_up.device)
    check(lib().fg_silu_mul(ptr(gate_up), ptr(out), dtype_code(gate_up.dtype), M, F, stream()), "silu_mul")
    return out


def gemm_generic(a: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None,
                 out_dtype: Optional[torch.dtype] = None, accumulate: bool = False) -> torch.Tensor:
    """out[m, n] (+)= sum_k a[m, k] * w[n, k] on the FMA units with f32 accumulation."""
    require_cuda(a, w, out)
    M, K = a.shape
    N, K2 = w.shape
    if K != K2:
        raise KernelError(f"gemm: a is [{M}, {K}] but w is [{N}, {K2}]")
    if a.stride(1) != 1 or w.stride(1) != 1:
        raise KernelError("gemm: the reduction dimension must be contiguous in both operands")
    if out is None:
        if accumulate:
            raise KernelError("gemm: accumulate needs the tensor to accumulate into")
        out = torch.empty((M, N), dtype=out_dtype or a.dtype, device=a.device)
    if out.shape != (M, N) or out.stride(1) != 1:
        raise KernelError(f"gemm: out must be [{M}, {N}] with contiguous rows")
    if accumulate and out.dtype != torch.float32:
        raise KernelError("gemm: the residual sum is 32-bit; accumulate needs a float32 output")
    check(lib().fg_gemm_generic(ptr(a), dtype_code(a.dtype), a.stride(0), ptr(w), dtype_code(w.dtype), w.stride(0),
                                ptr(out), dtype_code(out.dtype), out.stride(0), int(accumulate), M, N, K, stream()),
          "gemm_generic")
    return out


def attention_generic(q: torch.Tensor, positions: torch.Tensor, row_seq: torch.Tensor,
                      block_table: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor,
                      n_heads: int, n_kv_heads: int, head_dim: int, scale: float, window: int = 0,
                      out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Each row attends to cache positions [max(0, pos - window + 1), pos] of its own sequence.

    q: [M, >= H*hd] (row stride free, heads first in the row); returns [M, H*hd].
    """
    require_cuda(q, positions, row_seq, block_table, k_pool, v_pool)
    M = q.shape[0]
    if q.stride(1) != 1 or q.shape[1] < n_heads * head_dim:
        raise KernelError("attention: q rows must be contiguous and hold every head")
    if k_pool.dtype != q.dtype or v_pool.dtype != q.dtype:
        raise KernelError("attention: q and the cache must share a dtype")
    if head_dim > 256:
        raise KernelError(f"attention: head_dim {head_dim} exceeds 256, the largest this kernel takes")
    if n_heads % n_kv_heads:
        raise KernelError(f"attention: {n_heads} heads are not a multiple of {n_kv_heads} KV heads")
    if out is None:
        out = torch.empty((M, n_heads * head_dim), dtype=q.dtype, device=q.device)
    check(lib().fg_attention_generic(ptr(q), q.stride(0), ptr(out), out.stride(0), dtype_code(q.dtype),
                                     ptr(_i32(positions, "positions")), ptr(_i32(row_seq, "row_seq")),
                                     ptr(_i32(block_table, "block_table")), block_table.shape[-1],
                                     ptr(k_pool), ptr(v_pool), M, n_heads, n_kv_heads, head_dim,
                                     k_pool.shape[2], float(scale), int(window), stream()),
          "attention_generic")
    return out


def attention(q: torch.Tensor, batch, block_table: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor,
              n_heads: int, n_kv_heads: int, head_dim: int, scale: float, window: int = 0) -> torch.Tensor:
    """Attention of a step's rows over the cache; picks the kernel by dtype, sizes and step shape."""
    from . import fast_attention
    if fast_attention.supported(q, k_pool, head_dim):
        if batch.single_token:
            return fast_attention.attention_decode(q, batch.positions, block_table, k_pool, v_pool, n_heads,
                                                   n_kv_heads, head_dim, scale, window)
        # Many new tokens: 128-row tiles on the tcgen05 tensor cores.  A few rows (a sequence fed in short pieces)
        # waste less of the mma.sync kernel's 64-row tile.
        prefill = (fast_attention.attention_prefill_tc
                   if head_dim in (64, 128) and batch.max_new * (n_heads // n_kv_heads) >= 64
                   and q.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0
                   else fast_attention.attention_prefill)
        return prefill(q, batch.cu_rows, batch.seq_start, block_table, k_pool, v_pool, batch.n_seq, batch.max_new,
                       n_heads, n_kv_heads, head_dim, scale, window)
    return attention_generic(q, batch.positions, batch.row_seq, block_table, k_pool, v_pool,
                             n_heads, n_kv_heads, head_dim, scale, window)


def rope_attention(qkv: torch.Tensor, batch, block_table: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor,
                   cos: torch.Tensor, sin: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int, scale: float,
                   window: int = 0, write_kv: bool = True) -> torch.Tensor:
    """Rotary encoding of q (and k), cache append (when ``write_kv``) and attention of a step's rows.
    A decode step in bfloat16 with head size 64 / 128 runs as one kernel; everything else as RoPE + append
    followed by the attention kernel the step's shape calls for."""
    from . import fast_attention
    if (write_kv and batch.single_token and fast_attention.supported(qkv, k_pool, head_dim)
            and qkv.stride(0) % 8 == 0 and qkv.data_ptr() % 16 == 0):
        out = fast_attention.attention_decode_fused(qkv, batch.positions, block_table, k_pool, v_pool, cos, sin,
                                                    n_heads, n_kv_heads, head_dim, scale, window)
        if out is not None:
            return out
    rope_append(qkv, batch.positions, batch.row_seq, block_table, k_pool, v_pool, cos, sin, n_heads, n_kv_heads,
                head_dim, write_kv=write_kv)
    return attention(qkv, batch, block_table, k_pool, v_pool, n_heads, n_kv_heads, head_dim, scale, window)


def argmax(logits: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Index of the first maximum of each row.  logits: [B, V] f32."""
    require_cuda(logits)
    B, V = logits.shape
    if logits.dtype != torch.float32 or logits.stride(1) != 1:
        raise KernelError("argmax: logits must be float32 with contiguous rows")
    if out is None:
        out = torch.empty((B,), dtype=torch.int32, device=logits.device)
    check(lib().fg_argmax(ptr(logits), B, V, logits.stride(0), ptr(out), stream()), "argmax")
    return out


def sample(logits: torch.Tensor, *, temp: float, top_k: int, top_p: float, repeat_penalty: float,
           repeat_last_n: int, seq_slot: torch.Tensor, rng: torch.Tensor,
           hist: Optional[torch.Tensor], hist_count: Optional[torch.Tensor],
           stop_ids: Optional[torch.Tensor], out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One token per row of ``logits`` ([B, V] f32, modified in place by the repeat penalty).

    ``seq_slot[b]`` names the row of ``rng`` ([n] int64 xorshift64* states, never zero) and of
    ``hist`` ([n, cap] int32 recent tokens, oldest first) / ``hist_count`` ([n] int32) that
    belongs to sequence b; the chosen token is appended to that history.
    """
    require_cuda(logits, seq_slot, rng, hist, hist_count, stop_ids)
    B, V = logits.shape
    if logits.dtype != torch.float32 or logits.stride(1) != 1:
        raise KernelError("sample: logits must be float32 with contiguous rows")
    if rng.dtype != torch.int64:
        raise KernelError("sample: rng states are int64")
    if top_k > 1024:
        raise KernelError(f"sample: top_k {top_k} exceeds 1024, the largest the sampler takes (0 turns top-k off)")
    if out is None:
        out = torch.empty((B,), dtype=torch.int32, device=logits.device)
    cap = 0 if hist is None else hist.shape[1]
    n_stop = 0 if stop_ids is None else stop_ids.numel()
    scratch = None
    if temp > 0 and top_k <= 128:
        # 4096 words a row: candidates of the two-stage top-k, or the state of the sampler without top-k (zero on entry)
        scratch = torch.zeros((B, 4096), dtype=torch.int64, device=logits.device)
    check(lib().fg_sample(ptr(logits), B, V, logits.stride(0), float(temp), int(top_k), float(top_p),
                          float(repeat_penalty), int(repeat_last_n), ptr(_i32(seq_slot, "seq_slot")), ptr(rng),
                          ptr(hist), cap, ptr(hist_count), ptr(stop_ids), n_stop, ptr(out), ptr(scratch), stream()),
          "sample")
    return out


def decode_advance(tokens: torch.Tensor, positions: torch.Tensor, next_tokens: torch.Tensor,
                   active: torch.Tensor) -> None:
    """tokens <- next_tokens; positions += 1 where active (all int32, same length)."""
    require_cuda(tokens, positions, next_tokens, active)
    check(lib().fg_decode_advance(ptr(_i32(tokens, "tokens")), ptr(_i32(positions, "positions")),
                                  ptr(_i32(next_tokens, "next_tokens")), ptr(_i32(active, "active")),
                                  tokens.numel(), stream()), "decode_advance")
