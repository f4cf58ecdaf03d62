"""GQAAttention(hidden_size, n_heads, n_kv_heads, head_dim, position, scale, window): grouped-query
attention over the paged cache.

Reference, per token (fastgguf.c): q, k, v projections in one fused pass (:4692-4696), rotary
encoding of q and k (:4702, :4718), K stored after rotation and V raw at the token's position
(:4720, :4738-4739), ``scale = 1/sqrt(head_dim)`` (:4744), each query head h attends with KV head
``h / (H / KV)`` (:4781) to positions ``[start, pos]`` (:4754-4758), softmax and value sum
(``attn_rows`` :3273-3326), output projection added onto the un-normalized input (:4860-4862).
A run that borrows the cache of an earlier entry computes only q and attends to the owner's
keys and values (the reference's shared-KV layers, :4745-4751).
"""
from __future__ import annotations

import math
from typing import Dict, Optional

import torch

from .. import ops
from .base import CacheRequest, LayerIO, Mixer, Runtime, TensorSpec, register_mixer
from .linear import Linear


class GQAAttention(Mixer):
    #: takes a ``DeferredNorm`` as input and can start the next norm from its output projection
    supports_deferred_norm = True

    def __init__(self, runtime: Runtime, hidden_size: int, n_heads: int, n_kv_heads: int, head_dim: int,
                 position=None, scale: Optional[float] = None, window: Optional[int] = None):
        super().__init__(runtime)
        if n_heads % n_kv_heads:
            raise ValueError(f"{n_heads} heads are not a multiple of {n_kv_heads} KV heads")
        self.hidden_size, self.n_heads, self.n_kv_heads, self.head_dim = hidden_size, n_heads, n_kv_heads, head_dim
        self.q_dim, self.kv_dim = n_heads * head_dim, n_kv_heads * head_dim
        self.position = position
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(head_dim)
        self.window = window
        self.qkv: Optional[Linear] = None
        self.q_only: Optional[Linear] = None
        self.o: Optional[Linear] = None

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        E = self.hidden_size
        return {
            "q_proj.weight": TensorSpec((self.q_dim, E)),
            "k_proj.weight": TensorSpec((self.kv_dim, E)),
            "v_proj.weight": TensorSpec((self.kv_dim, E)),
            "o_proj.weight": TensorSpec((E, self.q_dim)),
        }

    def cache_request(self) -> Optional[CacheRequest]:
        return CacheRequest(self.n_kv_heads, self.head_dim, self.window)

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        parts = [tensors["q_proj.weight"], tensors["k_proj.weight"], tensors["v_proj.weight"]]
        dt = parts[0].dtype if all(p.dtype == parts[0].dtype for p in parts) else torch.float32
        fused = torch.cat([p.to(dt) for p in parts], dim=0).contiguous()
        self.qkv = Linear(fused)
        self.q_only = self.qkv.rows(0, self.q_dim)
        self.o = Linear(tensors["o_proj.weight"].contiguous())

    def forward(self, xn, batch, io: LayerIO, residual: torch.Tensor, emit_norm=None):
        proj = self.qkv if io.write_cache else self.q_only
        qkv = proj.forward(xn, out_dtype=self.runtime.dtype)
        table = batch.block_tables[io.group]
        if self.position is None:
            raise NotImplementedError("attention without a position encoding is not built")
        attn = ops.rope_attention(qkv, batch, table, io.k_pool, io.v_pool, self.position.cos, self.position.sin,
                                  self.n_heads, self.n_kv_heads, self.head_dim, self.scale, self.window or 0,
                                  write_kv=io.write_cache)
        if emit_norm is None:
            self.o.forward(attn, out=residual, accumulate=True)
            return None
        return self.o.forward(attn, out=residual, accumulate=True, emit_norm=emit_norm)[1]


register_mixer("gqa_attention", GQAAttention)
