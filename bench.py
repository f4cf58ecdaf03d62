#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on one GPU, as one JSON line.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--model 1b|3b|8b] [--dtype bfloat16|float32]
                    [--layers L] [--no-points] [--no-prefill] [--impl reference]

Default run: the layer sizes of Llama 3.2 1B with random weights, bfloat16, a batch of 8 sequences with random
prompts of unequal lengths 128..1024, context 4096.  ``--model 3b``: prompts 64..2048, context 4096; ``--model 8b``:
context 8192 with prompts that end shortly before it, so that decoding runs near the full context.  A "step" is one
decode step of the whole batch.  ``value`` is decoded tokens a second timed on the device (CUDA events around K
graph-replayed steps, the median of 5 such regions); ``e2e`` is the same through ``Engine.generate`` with host token
lists in and out; ``prefill`` is one step of 2,048 prompt tokens; ``roofline`` divides the bytes a decode step has to
read (every weight once, the cache of the live requests) by its time; ``points`` holds decode at batch 1 and 64, and
at the headline batch with the reference's default sampler instead of greedy; ``points_detail`` what each of them was
made of.  Every step reads gigabytes of weights, far more than the 126 MB L2, so no flush is needed between timed steps.
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
#: per model: context, shortest and longest prompt of the decode workload
WORKLOADS = {"1b": (4096, 128, 1024), "3b": (4096, 64, 2048), "8b": (8192, 7168, 7680)}
PREFILL_TOKENS = 2048
REPEATS = 5
#: peak of the FP32 FMA units: 148 SMs x 128 lanes x 2 flops at the maximum SM clock (no measured figure exists)
FP32_TFLOPS = 148 * 128 * 2 * 1.965e9 / 1e12
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


def layer_weight_bytes(c, size=2):
    E, F = c["hidden_size"], c["intermediate_size"]
    Q = c["num_attention_heads"] * c["head_dim"]
    D = c["num_key_value_heads"] * c["head_dim"]
    return size * (E * (Q + 2 * D) + Q * E + 3 * E * F + 2 * E)


def decode_step_bytes(c, layers, context_tokens, size=2):
    """Bytes one decode step must read: every weight it uses once, and the cache of the live requests
    (``size`` bytes an element: 2 in bfloat16, 4 on the 32-bit path)."""
    head = size * c["vocab_size"] * c["hidden_size"] + size * c["hidden_size"]      # the head matrix (tied or not) is read once
    kv = context_tokens * layers * 2 * c["num_key_value_heads"] * c["head_dim"] * size
    return layers * layer_weight_bytes(c, size) + head + kv


def prefill_flops(c, layers, T):
    E, F = c["hidden_size"], c["intermediate_size"]
    Q = c["num_attention_heads"] * c["head_dim"]
    D = c["num_key_value_heads"] * c["head_dim"]
    gemm = 2 * T * (E * (Q + 2 * D) + Q * E + 3 * E * F)
    attn = 2 * 2 * (T * (T + 1) // 2) * Q          # causal QK^T and PV
    return layers * (gemm + attn) + 2 * c["vocab_size"] * E


def reference_arm(args):
    """The reference has no installer and no GPU path; see baseline/reference_arm.py for what can be run of it."""
    try:
        sys.path.insert(0, os.path.join(ROOT, "baseline"))
        import reference_arm as arm
    except ImportError:
        return {"impl": "reference", "unavailable":
                "lawnak/FastGGUF is one C file with no setup.py or pyproject.toml: pip cannot install it into "
                "baseline/_ref, and it has no CUDA path to run on a B200"}
    return arm.run(args, LLAMA_3_2_1B)


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=16)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the configuration (named in config)")
    ap.add_argument("--model", default="1b", choices=sorted(MODELS), help="layer sizes (default: the 1B configuration)")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"], help="float32: the true 32-bit path")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-points", action="store_true", help="skip the batch 1 / 64 points")
    ap.add_argument("--no-prefill", action="store_true", help="skip the prefill measurement")
    ap.add_argument("--no-e2e", action="store_true", help="skip the end-to-end measurement")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps(reference_arm(args)))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2

    import numpy as np
    import torch
    from fastgguf_b200.engine.api import Engine
    from fastgguf_b200.engine.batch import StepEntry
    from fastgguf_b200.registry import config_from_dict
    from fastgguf_b200.sampling import SamplingParams

    W = max(3, args.warmup)
    K = args.steps
    model_name, base = MODELS[args.model]
    context, prompt_min, prompt_max = WORKLOADS[args.model]
    c = dict(base)
    full_layers = c["num_hidden_layers"]
    if args.layers:
        c["num_hidden_layers"] = args.layers
    layers = c["num_hidden_layers"]
    cfg = config_from_dict(c)
    pk = peaks()
    f32 = args.dtype == "float32"
    size = 4 if f32 else 2
    points_at = () if args.no_points else ((1, 8) if f32 else (1, 64))
    max_batch = max([args.batch, *points_at])
    # the cache holds what the largest batch needs: every sequence up to its longest prompt plus the decoded tokens
    per_seq = min(context, prompt_max + W + K * REPEATS + 128)
    per_seq = (per_seq + 63) // 64 * 64
    engine = Engine.from_random(cfg, 0, dtype=args.dtype, max_tokens=max(max_batch * per_seq, PREFILL_TOKENS + 64),
                                max_batch=max_batch, max_seq_len=context, verbose=True)
    info = engine.info()
    stream = torch.cuda.ExternalStream(engine.stream)
    rng = np.random.default_rng(0)
    params = SamplingParams(temp=0.0)

    def make_prompts(n, steps_ahead):
        hi = min(prompt_max, context - steps_ahead - 1)
        lo = min(prompt_min, hi)
        return [rng.integers(0, c["vocab_size"], size=int(L)).tolist() for L in rng.integers(lo, hi + 1, size=n)]

    def timed_decode(batch, warmup, steps, repeats, params=params):
        """(median ms per step over `repeats` regions of `steps` steps, launches per step, mean context tokens)."""
        prompts = make_prompts(batch, warmup + steps * repeats)
        session = engine.session(prompts, params)
        try:
            live = list(range(batch))
            for _ in range(warmup):
                session.advance(live)
            engine.check_device()
            ctx0 = sum(engine.cache.length(s) for s in session.slots)
            times = []
            for _ in range(repeats):
                t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                t0.record(stream)
                for _ in range(steps):
                    session.advance(live)
                t1.record(stream)
                t1.synchronize()
                times.append(t0.elapsed_time(t1) / steps)
            engine.check_device()                     # a number from a broken pipeline is no number
            ms = sorted(times)[len(times) // 2]
            mean_ctx = ctx0 + batch * (steps * repeats + 1) / 2.0
        finally:
            session.close()
        return ms, session.launches_per_step, mean_ctx, times

    # ---- headline: decode at --batch, device-timed, clocks sampled meanwhile
    timed_decode(args.batch, 3, 3, 1)                   # records the graph, warms everything up
    with ClockSampler() as clocks:
        ms_step, launches, mean_ctx, times = timed_decode(args.batch, W, K, REPEATS)
    value = args.batch * 1000.0 / ms_step
    step_bytes = decode_step_bytes(c, layers, mean_ctx, size)
    achieved = step_bytes / (ms_step * 1e-3) / 1e9

    rec = {
        "metric": "decode tokens/s (%s, %s, batch %d, context %d)" % (model_name, "fp32" if f32 else "bf16", args.batch, context),
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": K, "warmup": W,
        "ms_per_step": round(ms_step, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "fp32" if f32 else "bf16", "data": "synthetic: random weights N(0, 0.02), uniform random token ids",
        "config": {
            "model": model_name, "layers": layers, "layers_full": full_layers, "hidden": c["hidden_size"],
            "heads": c["num_attention_heads"], "kv_heads": c["num_key_value_heads"], "head_dim": c["head_dim"],
            "d_ff": c["intermediate_size"], "vocab": c["vocab_size"], "tied_head": c["tie_word_embeddings"],
            "rope": "llama3 x%g theta 5e5" % c["rope_scaling"]["factor"],
            "global_batch": args.batch, "seq_len": context, "prompt_lens": "%d-%d unequal" % (prompt_min, prompt_max),
            "mean_context": round(mean_ctx / args.batch, 1), "parallelism": "single GPU",
            "l2": "inputs larger than L2: each step reads %.2f GB" % (step_bytes / 1e9),
            "peaks": pk["source"], "timing": "median of %d regions of %d steps" % (REPEATS, K),
            "cache_mib": round(info["cache_bytes"] / 2 ** 20, 1),
        },
        "clocks": clocks.summary(),
        "gpu_launches": int(launches * K) if launches else None,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
    }

    if not args.no_e2e:
        # ---- end to end through Engine.generate: host token lists in, host token lists out
        prompts = make_prompts(args.batch, K + 8)
        engine.generate(prompts, temp=0, max_tokens=4, ignore_eos=True)
        s0 = engine.stats()
        t = time.perf_counter()
        engine.generate(prompts, temp=0, max_tokens=1, ignore_eos=True)
        t_first = time.perf_counter() - t
        s_mid = engine.stats()
        t = time.perf_counter()
        out = engine.generate(prompts, temp=0, max_tokens=K + 1, ignore_eos=True)
        t_all = time.perf_counter() - t
        assert all(len(o.tokens) == K + 1 for o in out)
        e2e = args.batch * K / max(t_all - t_first, 1e-9)
        s1 = engine.stats()
        n_steps = max(1, s1["steps"] - s_mid["steps"])
        rec["e2e"] = {"value": round(e2e, 1), "unit": "tokens/s",
                      "h2d_bytes_per_step": round((s1["h2d_bytes"] - s_mid["h2d_bytes"]) / n_steps, 1),
                      "d2h_bytes_per_step": round((s1["d2h_bytes"] - s_mid["d2h_bytes"]) / n_steps, 1)}

    if not args.no_prefill:
        # ---- prefill of 2,048 tokens in one step
        toks = rng.integers(0, c["vocab_size"], size=PREFILL_TOKENS).tolist()
        times = []
        for i in range(3 + 5):
            slot = engine.acquire()
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            engine.check_device()
            t0.record(stream)
            engine.step_host([StepEntry(slot, toks, [PREFILL_TOKENS - 1])])
            t1.record(stream)
            t1.synchronize()
            engine.release(slot)
            if i >= 3:
                times.append(t0.elapsed_time(t1))
        pms = sorted(times)[len(times) // 2]
        fl = prefill_flops(c, layers, PREFILL_TOKENS)
        peak = FP32_TFLOPS if f32 else pk["bf16_tflops"]
        rec["prefill"] = {"value": round(PREFILL_TOKENS / (pms * 1e-3), 1), "tokens": PREFILL_TOKENS, "ms": round(pms, 3),
                          "frac": round(fl / (pms * 1e-3) / 1e12 / peak, 4)}
        if f32:
            rec["prefill"]["peak_tflops"] = round(FP32_TFLOPS, 1)
    if points_at:
        points, detail = {}, {}
        for b in points_at:
            timed_decode(b, 3, 3, 1)
            with ClockSampler() as pc:
                ms_b, _, ctx_b, _ = timed_decode(b, W, min(K, 128), REPEATS)
            bytes_b = decode_step_bytes(c, layers, ctx_b, size)
            points["decode_b%d" % b] = round(b * 1000.0 / ms_b, 1)
            detail["decode_b%d" % b] = {"ms_per_step": round(ms_b, 4), "mean_context": round(ctx_b / b, 1), "bytes": int(bytes_b),
                                        "frac": round(bytes_b / (ms_b * 1e-3) / 1e9 / pk["hbm_gbs"], 4),
                                        "sm_mhz": pc.summary()["sm_mhz"], "reasons": pc.summary()["reasons"]}
        # the headline batch again with the reference's default sampler (temperature 1, top-k 64, top-p 0.95) instead of greedy
        sampled = SamplingParams(temp=1.0, top_k=64, top_p=0.95, seed=1)
        timed_decode(args.batch, 3, 3, 1, sampled)
        ms_s, _, ctx_s, _ = timed_decode(args.batch, W, min(K, 128), REPEATS, sampled)
        points["decode_b%d_sampled" % args.batch] = round(args.batch * 1000.0 / ms_s, 1)
        detail["decode_b%d_sampled" % args.batch] = {"ms_per_step": round(ms_s, 4), "mean_context": round(ctx_s / args.batch, 1),
                                                     "sampler": "temp 1.0 top_k 64 top_p 0.95"}
        rec["points"] = points
        rec["points_detail"] = detail
    print(json.dumps(rec))
    return 0


if __name__ == "__main__":
    sys.exit(main())
