"""Seeded random configurations and batch shapes, engine against the plain implementation.

Every size is drawn: head size (64 / 128 for the tensor-core attention kernels, 32 / 48 for the plain ones), heads
and groups, widths that are and are not multiples of 64, the vocabulary, layers, rotary scaling, tied or untied
head; then a batch of unequal prompts (a single token, page edges 63 / 64 / 65, several pages; now and then more
than 64 sequences, which takes the decode contraction in blocks of tokens), logits wanted at a few places, and
decode steps during which sequences leave the batch."""
import numpy as np
import pytest
import torch

import plain_llama
from helpers import TOL, make_model_dir, rel_err

pytestmark = pytest.mark.gpu


def draw_case(seed):
    rng = np.random.default_rng(seed)
    hd = int(rng.choice([64, 128, 64, 128, 32, 48]))
    KV = int(rng.choice([1, 2, 3, 4]))
    G = int(rng.choice([1, 2, 3, 4, 5, 8] if hd >= 64 else [1, 2, 4]))
    scaling = None if rng.random() < 0.5 else {
        "rope_type": "llama3", "factor": float(rng.choice([2.0, 8.0])), "low_freq_factor": 1.0, "high_freq_factor": 4.0,
        "original_max_position_embeddings": int(rng.choice([32, 256]))}
    cfg = {"architectures": ["LlamaForCausalLM"], "model_type": "llama", "hidden_size": int(rng.choice([128, 192, 256, 320, 200, 136])),
           "num_hidden_layers": int(rng.integers(1, 4)), "num_attention_heads": KV * G, "num_key_value_heads": KV, "head_dim": hd,
           "intermediate_size": int(rng.choice([128, 192, 320, 448, 100, 264])), "vocab_size": int(rng.integers(50, 700)),
           "rms_norm_eps": float(rng.choice([1e-5, 1e-6])), "rope_theta": float(rng.choice([1e4, 5e5])), "rope_scaling": scaling,
           "max_position_embeddings": 4096, "tie_word_embeddings": bool(rng.random() < 0.5), "hidden_act": "silu", "eos_token_id": 2}
    many = rng.random() < 0.25
    B = int(rng.integers(60, 131)) if many else int(rng.integers(1, 7))
    lens = [int(rng.choice([1, 3, 17] if many else [1, 3, 17, 63, 64, 65, 130, 200, 333])) for _ in range(B)]
    dtype = "bfloat16" if rng.random() < 0.8 else "float32"
    return rng, cfg, lens, int(rng.integers(1, 6)), dtype


@pytest.mark.parametrize("seed", [1003, 1005, 1014, 2007, 2016, 2028, 3002, 3011, 3020, 3033, 3041, 3055])
def test_random_configuration(tmp_path, seed):
    from fastgguf_b200.engine.api import Engine
    from fastgguf_b200.engine.batch import StepEntry
    rng, cfg_dict, lens, n_dec, dtype = draw_case(seed)
    model_dir = make_model_dir(tmp_path, cfg_dict, seed, torch.bfloat16)
    cfg, W = plain_llama.read_model_folder(model_dir)
    B, V = len(lens), cfg_dict["vocab_size"]
    engine = Engine.from_dir(model_dir, dtype=dtype, max_tokens=B * 640, max_batch=B, max_seq_len=600)
    toks = [[int(t) for t in rng.integers(0, V, size=n + n_dec)] for n in lens]
    want = [plain_llama.plain_forward(cfg, W, t).numpy() for t in toks]
    slots = [engine.acquire() for _ in range(B)]
    places = [sorted(set([0, n - 1] + [int(x) for x in rng.integers(0, n, size=2)])) for n in lens]
    got = engine.step([StepEntry(s, t[:n], w) for s, t, n, w in zip(slots, toks, lens, places)]).float().cpu().numpy()
    row = 0
    for b in range(B):
        for w in places[b]:
            assert rel_err(got[row], want[b][w]) < TOL[dtype], (seed, "prompt", b, w)
            row += 1
    alive = list(range(B))
    for d in range(n_dec):
        got = engine.step([StepEntry(slots[b], [toks[b][lens[b] + d]], [0]) for b in alive]).float().cpu().numpy()
        for i, b in enumerate(alive):
            assert rel_err(got[i], want[b][lens[b] + d]) < TOL[dtype], (seed, "decode", d, b)
        if len(alive) > 1 and rng.random() < 0.4:
            engine.release(slots[alive.pop(int(rng.integers(len(alive))))])
    for b in alive:
        engine.release(slots[b])
    engine.cache.check()
