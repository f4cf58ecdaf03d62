"""Timings of single kernels at sizes other than the engine's defaults.

    python -m fastgguf_b200.kernel_bench attention_prefill [--head-dim 64] [--heads 32] [--kv-heads 8]
    python -m fastgguf_b200.kernel_bench attention_decode  [--head-dim 64] [--heads 32] [--kv-heads 8]
    python -m fastgguf_b200.kernel_bench gemm [--hidden 2048] [--qkv 3072] [--ffn 8192]
    python -m fastgguf_b200.kernel_bench prompt_steps [--hidden 2048 --layers 16 --heads 32 --kv-heads 8 --head-dim 64
                                                       --ffn 8192 --vocab 128256]

Each line is one shape: the median of CUDA-event timings after warm-up launches, the work it stands for and the
fraction of the measured peak (``MEASURED_PEAKS.json`` beside the package's parent folder if present, else 6,650 GB/s
and 1,590 TFLOP/s).  The decode-attention and contraction timings write a buffer larger than L2 between launches; the
prefill attention is timed back to back (its K and V exceed L2 only at the longest prompts, as in a real prompt step).
A timing of one launch carries the launch itself (a few microseconds), which a graph-replayed step hides.
``prompt_steps`` is the whole engine instead: one prompt of 1 to 4,096 tokens through a model of random weights with
the given layer sizes (defaults: Llama 3.2 1B), host tokens in, the last position's logits out.
"""
import argparse
import json
import os

import torch

from .ops import fast_attention, fast_gemm

PAGE = 64


def _peaks():
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    hbm, tf = 6650.0, 1590.0
    try:
        with open(path) as f:
            d = json.load(f)
        hbm, tf = float(d.get("hbm_gbs", hbm)), float(d.get("bf16_tflops", tf))
    except (OSError, ValueError):
        pass
    return hbm, tf


class _Timer:
    def __init__(self, flush: bool):
        self.flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda") if flush else None

    def __call__(self, fn, warm=3, n=8):
        for _ in range(warm):
            fn()
        torch.cuda.synchronize()
        if self.flush is None:
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(n):
                fn()
            b.record()
            torch.cuda.synchronize()
            return a.elapsed_time(b) / n * 1e3
        ts = []
        for _ in range(n):
            self.flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b) * 1e3)
        return sorted(ts)[len(ts) // 2]


def _pools(n_seq, tokens, kv_heads, head_dim):
    pages_seq = (tokens + PAGE - 1) // PAGE
    n_pages = n_seq * pages_seq + 1
    k_pool = torch.randn(n_pages, kv_heads, PAGE, head_dim, device="cuda", dtype=torch.bfloat16)
    v_pool = torch.randn(n_pages, kv_heads, PAGE, head_dim, device="cuda", dtype=torch.bfloat16)
    table = (torch.randperm(n_pages - 1, device="cuda").to(torch.int32) + 1).view(n_seq, pages_seq).contiguous()
    return k_pool, v_pool, table


def attention_prefill(args):
    """Whole prompts from position 0: one sequence of each length, then eight of 2,048 tokens."""
    _, tf = _peaks()
    H, KV, hd = args.heads, args.kv_heads, args.head_dim
    time = _Timer(flush=False)
    for n_seq, T in [(1, 2048), (1, 4096), (1, 8192), (1, 16384), (1, 32768), (8, 2048)]:
        k_pool, v_pool, table = _pools(n_seq, T, KV, hd)
        q = torch.randn(n_seq * T, H * hd, device="cuda", dtype=torch.bfloat16)
        cu = torch.arange(0, n_seq + 1, dtype=torch.int32, device="cuda") * T
        start = torch.zeros(n_seq, dtype=torch.int32, device="cuda")
        out = torch.empty_like(q)
        us = time(lambda: fast_attention.attention_prefill_tc(q, cu, start, table, k_pool, v_pool, n_seq, T, H, KV, hd,
                                                              hd ** -0.5, 0, out=out), warm=2, n=5 if T >= 16384 else 20)
        if fast_attention.prefill_tc_error():
            raise RuntimeError("a bounded wait of the prefill attention ran out")
        flops = 4.0 * hd * H * n_seq * (T * (T + 1) / 2)
        print(f"attention_prefill head_dim {hd} heads {H} kv_heads {KV} sequences {n_seq} tokens {T:6d}: {us:10.1f} us  "
              f"{flops / us / 1e6:7.1f} TFLOP/s  {flops / us / 1e6 / tf:5.3f} of measured bf16", flush=True)


def attention_decode(args):
    """One new token per sequence over a cache of `context` tokens; bytes = the K and V the step has to read."""
    hbm, _ = _peaks()
    H, KV, hd = args.heads, args.kv_heads, args.head_dim
    time = _Timer(flush=True)
    for B, ctx in [(1, 1024), (1, 4096), (1, 16384), (1, 65536), (1, 131072), (8, 1024), (8, 4096), (8, 16384),
                   (8, 65536), (64, 512), (64, 2048), (64, 8192)]:
        k_pool, v_pool, table = _pools(B, ctx, KV, hd)
        q = torch.randn(B, H * hd, device="cuda", dtype=torch.bfloat16)
        pos = torch.full((B,), ctx - 1, dtype=torch.int32, device="cuda")
        out = torch.empty(B, H * hd, device="cuda", dtype=torch.bfloat16)
        splits = fast_attention.decode_splits(B, H, KV, table.shape[1], hd)
        us = time(lambda: fast_attention.attention_decode(q, pos, table, k_pool, v_pool, H, KV, hd, hd ** -0.5, 0, out=out))
        nbytes = B * ctx * KV * hd * 2 * 2
        print(f"attention_decode head_dim {hd} batch {B:3d} context {ctx:6d} splits {splits:3d}: {us:8.1f} us  "
              f"{nbytes / 1e6:8.1f} MB  {nbytes / us / 1e3:7.0f} GB/s  {nbytes / us / 1e3 / hbm:5.2f} of measured HBM", flush=True)


def gemm(args):
    """The four projections of a layer over row counts, beside torch.matmul (cuBLAS, plain bf16 output) for scale:
    the residual-add and SiLU forms do more than the library call they stand beside."""
    _, tf = _peaks()
    E, QKV, F = args.hidden, args.qkv, args.ffn
    time = _Timer(flush=True)
    for M in (8, 64, 128, 256, 512, 1024, 2048, 4096, 8192):
        cells = []
        for label, N, K, kw in [("qkv", QKV, E, {}), ("o+residual", E, E, {"accumulate": True}),
                                ("gate/up+silu", 2 * F, E, {"silu": True}), ("down+residual", E, F, {"accumulate": True})]:
            a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
            w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.02
            out = torch.zeros(M, N, device="cuda", dtype=torch.float32) if kw.get("accumulate") else None
            us = time(lambda: fast_gemm.gemm_tc(a, w, out=out, **kw))
            wt = w.t()
            lib = time(lambda: torch.matmul(a, wt))
            flops = 2.0 * M * N * K
            cells.append(f"{label} {us:7.1f} us {flops / us / 1e6:6.0f} TFLOP/s {flops / us / 1e6 / tf:4.2f} (cuBLAS {lib:7.1f} us)")
        print(f"gemm rows {M:5d}: " + " | ".join(cells), flush=True)
    if fast_gemm.pipeline_error():
        raise RuntimeError("a bounded wait of a contraction ran out")


def prompt_steps(args):
    """Time to the first token's logits over prompt lengths: one sequence, one step, its slot given back after it."""
    import numpy as np
    from .engine.api import Engine
    from .engine.batch import StepEntry
    from .registry import config_from_dict
    cfg = {"architectures": ["LlamaForCausalLM"], "hidden_size": args.hidden, "num_hidden_layers": args.layers,
           "num_attention_heads": args.heads, "num_key_value_heads": args.kv_heads, "head_dim": args.head_dim,
           "intermediate_size": args.ffn, "vocab_size": args.vocab, "rms_norm_eps": 1e-5, "rope_theta": 500000.0,
           "max_position_embeddings": 8192, "tie_word_embeddings": True}
    engine = Engine.from_random(config_from_dict(cfg), 0, dtype="bfloat16", max_tokens=4096 + 64, max_batch=1, max_seq_len=4096)
    rng = np.random.default_rng(0)
    for T in (1, 16, 64, 65, 128, 129, 192, 256, 384, 512, 768, 1024, 1536, 2048, 4096):
        tokens = rng.integers(0, args.vocab, size=T).tolist()
        times = []
        for i in range(6):
            slot = engine.acquire()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            a.record()
            engine.step_host([StepEntry(slot, tokens, [T - 1])])
            b.record()
            torch.cuda.synchronize()
            engine.release(slot)
            if i >= 2:
                times.append(a.elapsed_time(b))
        ms = sorted(times)[len(times) // 2]
        print(f"prompt_steps tokens {T:5d}: {ms:8.3f} ms  {T / ms:9.1f} tokens/ms", flush=True)


def main(argv=None):
    ap = argparse.ArgumentParser(prog="python -m fastgguf_b200.kernel_bench", description=__doc__.split("\n\n")[0])
    sub = ap.add_subparsers(dest="what", required=True)
    for name in ("attention_prefill", "attention_decode"):
        p = sub.add_parser(name)
        p.add_argument("--head-dim", type=int, default=64, choices=(64, 128))
        p.add_argument("--heads", type=int, default=32)
        p.add_argument("--kv-heads", type=int, default=8)
    p = sub.add_parser("gemm")
    p.add_argument("--hidden", type=int, default=2048)
    p.add_argument("--qkv", type=int, default=3072)
    p.add_argument("--ffn", type=int, default=8192)
    p = sub.add_parser("prompt_steps")
    for name, default in (("hidden", 2048), ("layers", 16), ("heads", 32), ("kv-heads", 8), ("head-dim", 64), ("ffn", 8192),
                          ("vocab", 128256)):
        p.add_argument("--" + name, type=int, default=default)
    args = ap.parse_args(argv)
    if not torch.cuda.is_available():
        raise SystemExit("kernel_bench needs a GPU")
    {"attention_prefill": attention_prefill, "attention_decode": attention_decode, "gemm": gemm,
     "prompt_steps": prompt_steps}[args.what](args)


if __name__ == "__main__":
    main()
