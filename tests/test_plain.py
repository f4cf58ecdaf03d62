"""The plain implementation against the reference engine's own output, and properties of its parts
in the style of the reference's selftest (fastgguf.c:5414-5475 sampler, :5826-5869 attention,
:5921-5936 RoPE)."""
import json
import os

import numpy as np
import torch

import plain_llama as P

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def test_plain_matches_the_reference_engine():
    """tests/golden/tiny_ref_logits.f32 was written by the reference's forward() (make_golden.py)."""
    cfg, W = P.read_model_folder(os.path.join(GOLDEN, "tiny_model"))
    meta = json.load(open(os.path.join(GOLDEN, "tiny_tokens.json")))
    ref = np.fromfile(os.path.join(GOLDEN, "tiny_ref_logits.f32"), dtype="<f4").reshape(len(meta["tokens"]), -1)
    for dtype, tol in ((torch.float64, 5e-7), (torch.float32, 2e-6)):
        mine = P.plain_forward(cfg, W, meta["tokens"], dtype).double().numpy()
        assert np.abs(mine - ref).max() < tol * max(1.0, np.abs(ref).max()), dtype


def test_rmsnorm_formula():
    x = torch.tensor([[3.0, 4.0, 0.0, 0.0]], dtype=torch.float64)
    w = torch.tensor([1.0, 2.0, 3.0, 4.0], dtype=torch.float64)
    y = P.plain_rmsnorm(x, w, 0.0)
    assert torch.allclose(y, torch.tensor([[3.0, 8.0, 0.0, 0.0]], dtype=torch.float64) / 2.5)


def test_rope_keeps_norms_and_depends_on_distance_only():
    g = torch.Generator().manual_seed(0)
    q = torch.randn(1, 1, 16, generator=g, dtype=torch.float64)
    k = torch.randn(1, 1, 16, generator=g, dtype=torch.float64)
    div = [1.0] * 8

    def score(pq, pk):
        return (P.plain_rope(q, [pq], 10000.0, div) * P.plain_rope(k, [pk], 10000.0, div)).sum().item()
    assert abs(P.plain_rope(q, [37], 10000.0, div).norm().item() - q.norm().item()) < 1e-12
    assert abs(score(5, 2) - score(105, 102)) < 1e-9 and abs(score(5, 2) - score(5, 3)) > 1e-6
    assert torch.equal(P.plain_rope(q, [0], 10000.0, div), q)
    # a divisor of 2 at position 2p equals no divisor at position p (the reference's RoPE scale test)
    assert torch.allclose(P.plain_rope(q, [14], 10000.0, [2.0] * 8), P.plain_rope(q, [7], 10000.0, div), atol=1e-12)


def test_llama3_divisors_use_all_three_branches():
    cfg = {"rope_theta": 500000.0, "rope_scaling": {"rope_type": "llama3", "factor": 4.0, "low_freq_factor": 1.0,
                                                    "high_freq_factor": 4.0, "original_max_position_embeddings": 32}}
    d = P.plain_rope_divisors(cfg, 24)
    assert d[0] == 1.0 and d[-1] == 4.0 and any(1.0 < v < 4.0 for v in d)
    assert all(b >= a for a, b in zip(d, d[1:]))
    assert P.plain_rope_divisors({"rope_scaling": None}, 24) == [1.0] * 12


def test_attention_is_causal_and_grouped():
    g = torch.Generator().manual_seed(1)
    q = torch.randn(6, 4, 8, generator=g, dtype=torch.float64)
    k = torch.randn(6, 2, 8, generator=g, dtype=torch.float64)
    v = torch.randn(6, 2, 8, generator=g, dtype=torch.float64)
    out = P.plain_attention(q, k, v, 0.3)
    k2, v2 = k.clone(), v.clone()
    k2[4:] += 5.0; v2[4:] -= 3.0                                   # the future must not matter
    assert torch.equal(P.plain_attention(q, k2, v2, 0.3)[:4], out[:4])
    assert torch.allclose(out[0, 1], v[0, 0]) and torch.allclose(out[0, 2], v[0, 1])   # heads 0,1 -> kv 0; 2,3 -> kv 1
    win = P.plain_attention(q, k, v, 0.3, window=2)
    assert torch.equal(win[:2], out[:2]) and not torch.allclose(win[5], out[5])


def test_sampler_greedy_topk1_and_penalty():
    lg = np.array([0.1, 2.0, 2.0, -1.0], dtype=np.float32)
    kw = dict(top_p=0.95, repeat_penalty=1.0, repeat_last_n=64)
    assert P.plain_sample(lg, 1, [], temp=0.0, top_k=64, **kw)[0] == 1          # first maximum wins
    for s in range(1, 30):
        assert P.plain_sample(lg, s, [], temp=1.0, top_k=1, **kw)[0] == 1
    # the penalty divides positive logits once per distinct token and flips the winner (fastgguf.c:5453-5466)
    tok, _ = P.plain_sample(np.array([1.0, 3.0, 2.9], dtype=np.float32), 1, [1, 1, 1], temp=0.0, top_k=0, top_p=1.0,
                            repeat_penalty=1.2, repeat_last_n=64)
    assert tok == 2
    tok, _ = P.plain_sample(np.array([1.0, 3.0, 2.9], dtype=np.float32), 1, [1], temp=0.0, top_k=0, top_p=1.0,
                            repeat_penalty=1.2, repeat_last_n=64, stop_ids=(1,))
    assert tok == 1                                                               # stop tokens are exempt


def test_sampler_statistics():
    """Draws follow the probabilities {.5, .3, .2}; top-p 0.6 keeps {.625, .375, 0} (fastgguf.c:5426-5444)."""
    lg = np.log(np.array([0.5, 0.3, 0.2], dtype=np.float64)).astype(np.float32)
    state, n = 12345, 20000
    counts = np.zeros(3)
    for _ in range(n):
        tok, state = P.plain_sample(lg, state, [], temp=1.0, top_k=0, top_p=1.0, repeat_penalty=1.0, repeat_last_n=0)
        counts[tok] += 1
    assert np.abs(counts / n - [0.5, 0.3, 0.2]).max() < 0.015
    counts = np.zeros(3)
    for _ in range(n):
        tok, state = P.plain_sample(lg, state, [], temp=1.0, top_k=3, top_p=0.6, repeat_penalty=1.0, repeat_last_n=0)
        counts[tok] += 1
    assert np.abs(counts / n - [0.625, 0.375, 0.0]).max() < 0.015


def test_rng_is_xorshift64star():
    s, out = P.plain_rng_next(1)
    assert s == (1 ^ (1 << 25)) ^ ((1 ^ (1 << 25)) >> 27) and out == (s * 0x2545F4914F6CDD1D) % 2 ** 64
    s2, u = P.plain_rng_uniform(88172645463325252)
    assert 0.0 <= float(u) < 1.0 and s2 != 88172645463325252
