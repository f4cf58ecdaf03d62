"""The reference arm of ``bench.py --impl reference``: the UNMODIFIED lawnak/FastGGUF, on the CPU.

The reference is one C file with a Makefile, no Python package and no CUDA path (its GPU code is an OpenCL mat-vec
offload), so there is nothing to ``pip install``: ``install()`` copies its tree to ``baseline/_ref/src`` and builds it
with its own Makefile (``make portable CC=gcc``: one binary that carries AVX-512 / AVX2 / plain builds and picks one at
start).  ``run()`` then does what the reference's own ``tools/bench.py`` does (tools/bench.py:38-46): it starts
``fastgguf chat MODEL.gguf CTX --temp 0 --max-tokens N`` with a prompt on the standard input and reads the line
``[prompt: …s (… tok/s) | gen: N tok @ … tok/s]`` that the reference prints itself (fastgguf.c:5312-5314).

The model is this repository's random Llama-3.2-1B-shaped weights (same generator, same seed as the other arm), exported
as a BF16 GGUF under the reference's tensor names, with Q/K rows permuted from the halves rotary layout to the
adjacent-pair layout the reference uses for ``llama`` (fastgguf.c:3138-3139, :4198), the llama3 frequency divisors as
``rope_freqs.weight`` (:4278) and a byte-fallback vocabulary so that its tokenizer can read the prompt.

What the number is: decode tokens a second of ONE sequence on the CPU cores of the machine - the reference runs one
sequence at a time and has no batches - so ``same_config`` is false and the ratio against the B200 arm is context, not
a like-for-like comparison.  None of this repository's kernels or engine code runs in this arm; only its weight
generator makes the file.
"""
from __future__ import annotations

import json
import math
import os
import re
import shutil
import subprocess
import sys
import tempfile
import time

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
REF_DIR = os.path.join(HERE, "_ref")
#: the reference's binary; $FASTGGUF_REFERENCE_BINARY names another build of it
BINARY = os.environ.get("FASTGGUF_REFERENCE_BINARY") or os.path.join(REF_DIR, "src", "fastgguf")
PROMPT = "Write a short paragraph about the history of computing and why fast local inference matters."


def install(reference_tree: str) -> str:
    """Copy the reference tree as it is and build it with its own Makefile; returns the binary's path."""
    src = os.path.join(REF_DIR, "src")
    shutil.rmtree(src, ignore_errors=True)
    os.makedirs(REF_DIR, exist_ok=True)
    shutil.copytree(reference_tree, src)
    subprocess.run(["make", "portable", "CC=gcc"], cwd=src, check=True, stdout=subprocess.DEVNULL)
    return BINARY


def _divisors(cfg: dict, hd: int):
    """llama3 frequency divisors per rotary pair (ones without scaling), as GGUF files carry them."""
    rs = cfg.get("rope_scaling")
    out = [1.0] * (hd // 2)
    if not rs or rs.get("rope_type", "default") == "default":
        return out
    theta, factor = float(cfg["rope_theta"]), float(rs["factor"])
    low, high, orig = float(rs["low_freq_factor"]), float(rs["high_freq_factor"]), float(rs["original_max_position_embeddings"])
    for j in range(hd // 2):
        wavelen = 2.0 * math.pi * theta ** (2.0 * j / hd)
        if wavelen > orig / low:
            out[j] = factor
        elif wavelen >= orig / high:
            s = (orig / wavelen - low) / (high - low)
            out[j] = 1.0 / ((1.0 - s) / factor + s)
    return out


def export_gguf(model_dir: str, out_path: str) -> None:
    """A model folder of this repository (bfloat16 safetensors) as a BF16 GGUF the reference can load and chat with."""
    import numpy as np
    from gguf import GGMLQuantizationType, GGUFWriter, TokenType

    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    path = os.path.join(model_dir, "model.safetensors")
    with open(path, "rb") as f:
        hlen = int.from_bytes(f.read(8), "little")
        header = json.loads(f.read(hlen))
    data = np.memmap(path, dtype=np.uint8, mode="r", offset=8 + hlen)

    def tensor(name):                          # bfloat16 bits as uint16 [rows, cols]
        info = header[name]
        assert info["dtype"] == "BF16", (name, info["dtype"])
        b, e = info["data_offsets"]
        return np.frombuffer(data[b:e], dtype=np.uint16).reshape(info["shape"])

    def f32(name):
        return (tensor(name).astype(np.uint32) << 16).view(np.float32)

    E, L = cfg["hidden_size"], cfg["num_hidden_layers"]
    H, KV, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    V = cfg["vocab_size"]

    def adjacent(w, heads):                    # rows (j, j + hd/2) of a head -> rows (2j, 2j + 1)
        return np.ascontiguousarray(w.reshape(heads, 2, hd // 2, w.shape[1]).transpose(0, 2, 1, 3).reshape(heads * hd, -1))

    w = GGUFWriter(out_path, "llama")
    w.add_name("random weights, Llama-3.2-1B shapes")
    w.add_block_count(L)
    w.add_context_length(cfg["max_position_embeddings"])
    w.add_embedding_length(E)
    w.add_feed_forward_length(cfg["intermediate_size"])
    w.add_head_count(H)
    w.add_head_count_kv(KV)
    w.add_key_length(hd)
    w.add_value_length(hd)
    w.add_layer_norm_rms_eps(cfg["rms_norm_eps"])
    w.add_rope_freq_base(cfg["rope_theta"])
    w.add_rope_dimension_count(hd)
    # a vocabulary its tokenizer can read any text with: three controls, the 256 byte tokens, a space, filler
    tokens = ["<unk>", "<s>", "</s>"] + [f"<0x{b:02X}>" for b in range(256)] + ["▁"]
    tokens += [f"t{i}" for i in range(V - len(tokens))]
    types = [TokenType.CONTROL] * 3 + [TokenType.BYTE] * 256 + [TokenType.NORMAL] * (V - 259)
    w.add_tokenizer_model("llama")
    w.add_token_list(tokens)
    w.add_token_scores([0.0] * V)
    w.add_token_types(types)
    w.add_bos_token_id(1)
    w.add_eos_token_id(2)
    bf16 = GGMLQuantizationType.BF16
    w.add_tensor("token_embd.weight", tensor("model.embed_tokens.weight"), raw_dtype=bf16)
    if not cfg.get("tie_word_embeddings", False):
        w.add_tensor("output.weight", tensor("lm_head.weight"), raw_dtype=bf16)
    w.add_tensor("output_norm.weight", f32("model.norm.weight"))
    w.add_tensor("rope_freqs.weight", np.asarray(_divisors(cfg, hd), dtype=np.float32))
    for i in range(L):
        p, b = f"model.layers.{i}.", f"blk.{i}."
        w.add_tensor(b + "attn_norm.weight", f32(p + "input_layernorm.weight"))
        w.add_tensor(b + "attn_q.weight", adjacent(tensor(p + "self_attn.q_proj.weight"), H), raw_dtype=bf16)
        w.add_tensor(b + "attn_k.weight", adjacent(tensor(p + "self_attn.k_proj.weight"), KV), raw_dtype=bf16)
        w.add_tensor(b + "attn_v.weight", tensor(p + "self_attn.v_proj.weight"), raw_dtype=bf16)
        w.add_tensor(b + "attn_output.weight", tensor(p + "self_attn.o_proj.weight"), raw_dtype=bf16)
        w.add_tensor(b + "ffn_norm.weight", f32(p + "post_attention_layernorm.weight"))
        w.add_tensor(b + "ffn_gate.weight", tensor(p + "mlp.gate_proj.weight"), raw_dtype=bf16)
        w.add_tensor(b + "ffn_up.weight", tensor(p + "mlp.up_proj.weight"), raw_dtype=bf16)
        w.add_tensor(b + "ffn_down.weight", tensor(p + "mlp.down_proj.weight"), raw_dtype=bf16)
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file(progress=False)
    w.close()


def _unavailable(why: str) -> dict:
    return {"impl": "reference", "unavailable": why}


def run(args, cfg_dict: dict) -> dict:
    """One JSON-able record for ``bench.py --impl reference``."""
    if not os.path.exists(BINARY):
        return _unavailable("lawnak/FastGGUF is one C file with no setup.py or pyproject.toml (pip cannot install it) and no CUDA "
                            "path; its CPU build baseline/_ref/src/fastgguf (make portable) is not present on this machine")
    try:
        import gguf  # noqa: F401
    except ImportError:
        return _unavailable("the gguf package that writes the reference's model file is not installed on this machine")
    sys.path.insert(0, ROOT)
    from fastgguf_b200.registry import config_from_dict
    from fastgguf_b200.weights import write_random_model
    n_gen = max(8, min(int(args.steps), 64))
    ctx = 2048
    work = tempfile.mkdtemp(prefix="fg_reference_arm_")
    try:
        t0 = time.time()
        model_dir = write_random_model(config_from_dict(cfg_dict), 0, os.path.join(work, "model"), "bfloat16")
        gguf_path = os.path.join(work, "model.gguf")
        export_gguf(model_dir, gguf_path)
        shutil.rmtree(model_dir, ignore_errors=True)
        t_export = time.time() - t0
        env = dict(os.environ, FASTGGUF_GPU="off")
        best = None
        for _ in range(2):                       # the reference's own harness keeps the best of its runs (tools/bench.py:57)
            p = subprocess.run([BINARY, "chat", gguf_path, str(ctx), "--temp", "0", "--max-tokens", str(n_gen)],
                               input=PROMPT + "\n", capture_output=True, text=True, errors="replace", env=env, timeout=1500)
            out = p.stdout + p.stderr
            m = re.search(r"\[prompt: ([\d.]+)s \(([\d.]+) tok/s\) \| gen: (\d+) tok @ ([\d.]+) tok/s\]", out)
            if not m:
                return _unavailable("the reference ran but printed no timing line: " + " ".join(out[-300:].split()))
            rec = {"prompt_tok_s": float(m.group(2)), "gen_tokens": int(m.group(3)), "gen_tok_s": float(m.group(4))}
            if best is None or rec["gen_tok_s"] > best["gen_tok_s"]:
                best = rec
    except (OSError, subprocess.SubprocessError, ValueError) as e:
        return _unavailable(f"the reference's CPU run failed: {type(e).__name__}: {' '.join(str(e).split())[:200]}")
    finally:
        shutil.rmtree(work, ignore_errors=True)
    threads = os.environ.get("OMP_NUM_THREADS") or str(os.cpu_count())
    return {
        "impl": "reference", "metric": "decode tokens/s (Llama-3.2-1B shapes, bf16 weights, ONE sequence, CPU)",
        "value": best["gen_tok_s"], "unit": "tokens/s", "n_gpus": 0, "steps": best["gen_tokens"], "warmup": 0,
        "ms_per_step": round(1000.0 / max(best["gen_tok_s"], 1e-9), 3), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16 weights, f32 arithmetic", "same_config": False,
        "data": "synthetic: the same seeded random weights as the other arm, exported as a BF16 GGUF; the reference's own prompt",
        "config": {"model": "Llama-3.2-1B shapes", "global_batch": 1, "seq_len": ctx, "device": "CPU, %s threads" % threads,
                   "path": "fastgguf chat (stock), best of 2", "export_s": round(t_export, 1),
                   "note": "the reference runs one sequence on CPU cores; it has no batches and no CUDA path"},
        "e2e": {"value": best["gen_tok_s"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "prefill": {"value": best["prompt_tok_s"], "unit": "tokens/s"},
        "gpu_launches": 0,
    }


if __name__ == "__main__":
    if len(sys.argv) == 3 and sys.argv[1] == "--install":
        print(install(sys.argv[2]))
    else:
        print("usage: python baseline/reference_arm.py --install /path/to/reference/tree")
