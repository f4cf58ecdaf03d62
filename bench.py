#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on one GPU, as one JSON line.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--layers L] [--no-points] [--no-prefill]
                    [--impl reference]

Default run: the layer sizes of Llama 3.2 1B with random weights, bfloat16, a batch of 8
sequences with random prompts of unequal lengths 128..1024, context 4096.  A "step" is one
decode step of the whole batch.  ``value`` is decoded tokens a second timed on the device (CUDA
events around K graph-replayed steps); ``e2e`` is the same through ``Engine.generate`` with host
token lists in and out; ``prefill`` is one step of 2,048 prompt tokens; ``roofline`` divides the
bytes a decode step has to read (every weight once, the cache of the live requests) by its
time; ``points`` holds decode at batch 1 and 64.  Every step reads 2.5 GB of weights, far more
than the 126 MB L2, so no flush is needed between timed steps.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

LLAMA_3_2_1B = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "hidden_size": 2048, "num_hidden_layers": 16, "num_attention_heads": 32, "num_key_value_heads": 8,
    "head_dim": 64, "intermediate_size": 8192, "vocab_size": 128256, "rms_norm_eps": 1e-5,
    "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 8192},
    "max_position_embeddings": 131072, "tie_word_embeddings": True, "hidden_act": "silu",
    "bos_token_id": 128000, "eos_token_id": 128001,
}
LLAMA_3_2_3B = dict(LLAMA_3_2_1B, hidden_size=3072, num_hidden_layers=28, num_attention_heads=24, head_dim=128)
LLAMA_3_1_8B = dict(LLAMA_3_2_1B, hidden_size=4096, num_hidden_layers=32, num_attention_heads=32, head_dim=128,
                    intermediate_size=14336, tie_word_embeddings=False,
                    rope_scaling=dict(LLAMA_3_2_1B["rope_scaling"], factor=8.0))
MODELS = {"1b": ("Llama-3.2-1B shapes", LLAMA_3_2_1B), "3b": ("Llama-3.2-3B shapes", LLAMA_3_2_3B),
          "8b": ("Llama-3.1-8B shapes", LLAMA_3_1_8B)}
CONTEXT = 4096
PROMPT_MIN, PROMPT_MAX = 128, 1024
PREFILL_TOKENS = 2048
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            d = json.load(f)
        out = dict(FALLBACK_PEAKS)
        out.update({k: float(v) for k, v in d.items() if k in FALLBACK_PEAKS and isinstance(v, (int, float))})
        out["source"] = "measured"
        return out
    except (OSError, ValueError):
        return dict(FALLBACK_PEAKS, source="fallback")


class ClockSampler:
    """nvidia-smi clocks and throttle reasons, sampled while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows, self.proc = [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "--id=0", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "200"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *exc):
        if self.proc is not None:
            time.sleep(0.25)
            self.proc.terminate()

    def summary(self):
        sm = sorted(int(r[0]) for r in self.rows if r and r[0].isdigit())
        mx = [int(r[1]) for r in self.rows if len(r) > 1 and r[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) > 2 + i and r[2 + i].lower() == "active" for r in self.rows)]
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": reasons,
                "samples": len(sm)}


def layer_weight_bytes(c):
    E, F = c["hidden_size"], c["intermediate_size"]
    Q = c["num_attention_heads"] * c["head_dim"]
    D = c["num_key_value_heads"] * c["head_dim"]
    return 2 * (E * (Q + 2 * D) + Q * E + 3 * E * F + 2 * E)


def decode_step_bytes(c, layers, context_tokens):
    """Bytes one decode step must read: every weight it uses once, and the cache of the live requests."""
    head = 2 * c["vocab_size"] * c["hidden_size"] + 2 * c["hidden_size"]      # the head matrix (tied or not) is read once
    kv = context_tokens * layers * 2 * c["num_key_value_heads"] * c["head_dim"] * 2
    return layers * layer_weight_bytes(c) + head + kv


def prefill_flops(c, layers, T):
    E, F = c["hidden_size"], c["intermediate_size"]
    Q = c["num_attention_heads"] * c["head_dim"]
    D = c["num_key_value_heads"] * c["head_dim"]
    gemm = 2 * T * (E * (Q + 2 * D) + Q * E + 3 * E * F)
    attn = 2 * 2 * (T * (T + 1) // 2) * Q          # causal QK^T and PV
    return layers * (gemm + attn) + 2 * c["vocab_size"] * E


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=16)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the configuration (named in config)")
    ap.add_argument("--model", default="1b", choices=sorted(MODELS), help="layer sizes (default: the 1B configuration)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-points", action="store_true", help="skip the batch 1 / 64 points")
    ap.add_argument("--no-prefill", action="store_true", help="skip the prefill measurement")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "lawnak/FastGGUF is one C file with no setup.py or pyproject.toml: pip cannot install it "
                          "into baseline/_ref, and it has no CUDA path to run on a B200"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2

    import numpy as np
    import torch
    from fastgguf_b200 import ops
    from fastgguf_b200.engine.api import Engine
    from fastgguf_b200.engine.runner import DecodeSession
    from fastgguf_b200.registry import config_from_dict
    from fastgguf_b200.sampling import SamplingParams
    from fastgguf_b200.weights.random_init import random_tensors

    W = max(3, args.warmup)
    K = args.steps
    model_name, base = MODELS[args.model]
    c = dict(base)
    full_layers = c["num_hidden_layers"]
    if args.layers:
        c["num_hidden_layers"] = args.layers
    layers = c["num_hidden_layers"]
    cfg = config_from_dict(c)
    pk = peaks()
    torch.cuda.set_device(0)
    tensors = random_tensors(cfg, 0, torch.bfloat16, device="cuda")
    max_batch = max(args.batch, 1 if args.no_points else 64)
    engine = Engine.from_tensors(cfg, tensors, dtype="bfloat16", max_tokens=max_batch * CONTEXT, max_batch=max_batch,
                                 max_seq_len=CONTEXT)
    del tensors
    rng = np.random.default_rng(0)
    params = SamplingParams(temp=0.0)

    def make_prompts(n):
        return [rng.integers(0, c["vocab_size"], size=int(L)).tolist()
                for L in rng.integers(PROMPT_MIN, PROMPT_MAX + 1, size=n)]

    def timed_decode(batch, warmup, steps):
        """(ms per step, launches per step, mean context tokens over the timed steps)."""
        prompts = make_prompts(batch)
        backend = engine.backend(params, ())
        session = DecodeSession(backend, prompts)
        try:
            live = list(range(batch))
            for _ in range(warmup):
                session.advance(live)
            torch.cuda.synchronize()
            ctx0 = sum(engine.cache.length(s) for s in session.slots)
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0.record()
            for _ in range(steps):
                session.advance(live)
            t1.record()
            torch.cuda.synchronize()
            ops.raise_on_device_error("timed decode")      # a number from a broken pipeline is no number
            ms = t0.elapsed_time(t1) / steps
            mean_ctx = ctx0 + batch * (steps + 1) / 2.0
        finally:
            session.close()
        return ms, session.graph.launches_per_step, mean_ctx

    # ---- headline: decode at --batch, device-timed, clocks sampled meanwhile
    timed_decode(args.batch, 3, 3)                      # captures the graph, warms everything up
    with ClockSampler() as clocks:
        ms_step, launches, mean_ctx = timed_decode(args.batch, W, K)
    value = args.batch * 1000.0 / ms_step
    step_bytes = decode_step_bytes(c, layers, mean_ctx)
    achieved = step_bytes / (ms_step * 1e-3) / 1e9

    # ---- end to end through Engine.generate: host token lists in, host token lists out
    prompts = make_prompts(args.batch)
    backend = engine.backend(params, ())
    engine.generate(prompts, temp=0, max_tokens=4, ignore_eos=True)
    torch.cuda.synchronize()
    s0 = dict(backend.stats)
    t = time.perf_counter()
    engine.generate(prompts, temp=0, max_tokens=1, ignore_eos=True)
    t_first = time.perf_counter() - t
    t = time.perf_counter()
    out = engine.generate(prompts, temp=0, max_tokens=K + 1, ignore_eos=True)
    t_all = time.perf_counter() - t
    assert all(len(o.tokens) == K + 1 for o in out)
    e2e = args.batch * K / max(t_all - t_first, 1e-9)
    s1 = backend.stats
    n_steps = max(1, s1["steps"] - s0["steps"])
    e2e_rec = {"value": round(e2e, 1), "unit": "tokens/s", "h2d_bytes_per_step": round((s1["h2d_bytes"] - s0["h2d_bytes"]) / n_steps, 1),
               "d2h_bytes_per_step": round((s1["d2h_bytes"] - s0["d2h_bytes"]) / n_steps, 1)}

    rec = {
        "metric": "decode tokens/s (%s, bf16, batch %d, context %d)" % (model_name, args.batch, CONTEXT),
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": K, "warmup": W,
        "ms_per_step": round(ms_step, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: random weights N(0, 0.02), uniform random token ids",
        "config": {
            "model": model_name, "layers": layers, "layers_full": full_layers, "hidden": c["hidden_size"],
            "heads": c["num_attention_heads"], "kv_heads": c["num_key_value_heads"], "head_dim": c["head_dim"],
            "d_ff": c["intermediate_size"], "vocab": c["vocab_size"], "tied_head": c["tie_word_embeddings"],
            "rope": "llama3 x%g theta 5e5" % c["rope_scaling"]["factor"],
            "global_batch": args.batch, "seq_len": CONTEXT, "prompt_lens": "%d-%d unequal" % (PROMPT_MIN, PROMPT_MAX),
            "mean_context": round(mean_ctx / args.batch, 1), "parallelism": "single GPU",
            "l2": "inputs larger than L2: each step reads %.2f GB" % (step_bytes / 1e9),
            "peaks": pk["source"],
        },
        "clocks": clocks.summary(),
        "e2e": e2e_rec,
        "gpu_launches": int(launches * K) if launches else None,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
    }

    if not args.no_prefill:
        # ---- prefill of 2,048 tokens in one step
        toks = rng.integers(0, c["vocab_size"], size=PREFILL_TOKENS).tolist()
        from fastgguf_b200.engine.batch import StepEntry
        times = []
        for i in range(3 + 5):
            slot = engine.acquire()
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            t0.record()
            engine.step([StepEntry(slot, toks, [PREFILL_TOKENS - 1])])
            t1.record()
            torch.cuda.synchronize()
            ops.raise_on_device_error("timed prefill")
            engine.release(slot)
            if i >= 3:
                times.append(t0.elapsed_time(t1))
        pms = sorted(times)[len(times) // 2]
        fl = prefill_flops(c, layers, PREFILL_TOKENS)
        rec["prefill"] = {"value": round(PREFILL_TOKENS / (pms * 1e-3), 1), "tokens": PREFILL_TOKENS, "ms": round(pms, 3),
                          "frac": round(fl / (pms * 1e-3) / 1e12 / pk["bf16_tflops"], 4)}
    if not args.no_points:
        points = {}
        for b in (1, 64):
            timed_decode(b, 3, 3)
            ms_b, _, _ = timed_decode(b, W, min(K, 128))
            points["decode_b%d" % b] = round(b * 1000.0 / ms_b, 1)
        rec["points"] = points
    print(json.dumps(rec))
    return 0


if __name__ == "__main__":
    sys.exit(main())
