"""The measurement program's contract that needs no GPU: refusals, the reference arm's line, the roofline arithmetic."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import bench  # noqa: E402


def _run(*args, env=None):
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True, timeout=120,
                          env=dict(os.environ, **(env or {})))


def test_more_than_one_gpu_is_refused_with_one_line_and_code_2():
    r = _run("--gpus", "2")
    assert r.returncode == 2
    assert len(r.stdout.strip().splitlines()) == 1 and "one GPU" in r.stdout


def test_reference_arm_says_why_it_is_unavailable():
    """Where the reference's CPU build is absent the arm prints one line that says so and exits 0 (where it is present
    the arm runs it: a minute of CPU time, not part of this test)."""
    r = _run("--impl", "reference", "--gpus", "1", "--steps", "2", "--warmup", "1",
             env={"FASTGGUF_REFERENCE_BINARY": "/nonexistent/fastgguf"})
    assert r.returncode == 0
    rec = json.loads(r.stdout.strip().splitlines()[-1])
    assert rec["impl"] == "reference" and isinstance(rec["unavailable"], str) and "\n" not in rec["unavailable"]


def test_decode_bytes_and_prefill_flops_of_the_1b_shapes():
    c = bench.LLAMA_3_2_1B
    E, F, V, L = c["hidden_size"], c["intermediate_size"], c["vocab_size"], c["num_hidden_layers"]
    Q = c["num_attention_heads"] * c["head_dim"]
    D = c["num_key_value_heads"] * c["head_dim"]
    assert (E, F, V, L, Q, D) == (2048, 8192, 128256, 16, 2048, 512)
    per_layer = 2 * (E * (Q + 2 * D) + Q * E + 3 * E * F) + 2 * 2 * E          # bf16 matrices and the two f32-as-bf16 norms
    got = bench.decode_step_bytes(c, L, 0)
    # every matrix once (the tied head included), no cache yet: 2.47 GB
    assert abs(got - (L * per_layer + 2 * V * E)) <= 64 * 1024
    assert 2.4e9 < got < 2.5e9
    # the cache of the live requests: keys and values of every layer, bf16
    assert bench.decode_step_bytes(c, L, 1000) - got == 1000 * L * 2 * D * 2
    T = 2048
    fl = bench.prefill_flops(c, L, T)
    gemm = 2 * T * (E * (Q + 2 * D) + Q * E + 3 * E * F)
    attn = 2 * 2 * (T * (T + 1) // 2) * Q
    assert fl == L * (gemm + attn) + 2 * V * E
    assert 4.0e12 < fl < 4.6e12
