"""The full depth of the 1B configuration: 16 layers of its layer sizes (hidden 2048, 32 heads in groups of 4, head size
64, feed-forward 8192, llama3 rotary scaling, tied head) with a small vocabulary, bfloat16 engine against the plain
implementation in float32: three unequal prompts in one step, then four decoded tokens."""
import numpy as np
import pytest
import torch

import plain_llama
from helpers import make_model_dir, random_tokens, rel_err

pytestmark = pytest.mark.gpu

CONFIG = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama", "hidden_size": 2048, "num_hidden_layers": 16,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 64, "intermediate_size": 8192, "vocab_size": 1031,
    "rms_norm_eps": 1e-5, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 8192},
    "max_position_embeddings": 4096, "tie_word_embeddings": True, "hidden_act": "silu", "eos_token_id": 2,
}


def test_sixteen_layers_of_the_1b_sizes(tmp_path):
    from fastgguf_b200.engine.api import Engine
    from fastgguf_b200.engine.batch import StepEntry
    model_dir = make_model_dir(tmp_path, CONFIG, 21, "bfloat16")
    cfg, W = plain_llama.read_model_folder(model_dir)
    lens, extra = [70, 3, 130], 4
    seqs = [random_tokens(n + extra, cfg["vocab_size"], 400 + i) for i, n in enumerate(lens)]
    want = [plain_llama.plain_forward(cfg, W, s, torch.float32).numpy() for s in seqs]
    engine = Engine.from_dir(model_dir, dtype="bfloat16", max_tokens=1024, max_batch=4)
    slots = [engine.acquire() for _ in seqs]
    out = engine.step([StepEntry(sl, s[:n], list(range(n))) for sl, s, n in zip(slots, seqs, lens)]).cpu().numpy()
    got = [list(out[sum(lens[:i]):sum(lens[:i + 1])]) for i in range(len(seqs))]
    for k in range(extra):
        out = engine.step([StepEntry(sl, [s[n + k]], [0]) for sl, s, n in zip(slots, seqs, lens)]).cpu().numpy()
        for g, row in zip(got, out):
            g.append(row)
    for g, w in zip(got, want):
        assert rel_err(np.stack(g), w) < 3e-2
    engine.check_device()
