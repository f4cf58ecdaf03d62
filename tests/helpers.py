"""Tiny configurations and helpers shared by the tests.

The two tiny Llama configurations differ in every size and option: layers 2/3, width 64/144,
heads 4/6, KV heads 2/1, head size 16/24, vocabulary 256/509, eps 1e-5/1e-6,
theta 1e4/5e5, no rotary scaling / llama3 scaling, tied / untied head.
"""
import numpy as np
import torch

TINY_A = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "hidden_size": 64, "num_hidden_layers": 2, "num_attention_heads": 4, "num_key_value_heads": 2,
    "head_dim": 16, "intermediate_size": 192, "vocab_size": 256, "rms_norm_eps": 1e-5,
    "rope_theta": 10000.0, "rope_scaling": None, "max_position_embeddings": 512,
    "tie_word_embeddings": True, "hidden_act": "silu", "eos_token_id": 2,
}
TINY_B = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "hidden_size": 144, "num_hidden_layers": 3, "num_attention_heads": 6, "num_key_value_heads": 1,
    "head_dim": 24, "intermediate_size": 384, "vocab_size": 509, "rms_norm_eps": 1e-6,
    "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 4.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 32},
    "max_position_embeddings": 1024, "tie_word_embeddings": False, "hidden_act": "silu",
    "eos_token_id": [3, 5],
}
# head sizes the tensor-core attention kernels take: 64 with 4 query heads a KV head, 128 with 3
TINY_C = dict(TINY_A, hidden_size=256, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=1,
              head_dim=64, intermediate_size=448, vocab_size=300, max_position_embeddings=2048)
TINY_D = dict(TINY_B, hidden_size=200, num_hidden_layers=2, num_attention_heads=6, num_key_value_heads=2,
              head_dim=128, intermediate_size=320, vocab_size=333, max_position_embeddings=2048)
# sizes the tensor-core kernels refuse (reduction lengths that are no multiple of 8): the plain kernels in bfloat16
TINY_E = dict(TINY_A, hidden_size=100, num_attention_heads=3, num_key_value_heads=3, head_dim=16,
              intermediate_size=52, vocab_size=131, tie_word_embeddings=False)
TINY = {"a": (TINY_A, 0), "b": (TINY_B, 1), "c": (TINY_C, 2), "d": (TINY_D, 3), "e": (TINY_E, 4)}


def make_model_dir(tmp_path, cfg_dict, seed, dtype=torch.bfloat16):
    """Write a random model folder under tmp_path; returns its path."""
    from fastgguf_b200.registry import config_from_dict
    from fastgguf_b200.weights import write_random_model
    return write_random_model(config_from_dict(cfg_dict), seed, str(tmp_path), dtype)


def random_tokens(n, vocab, seed):
    rng = np.random.default_rng(seed)
    return [int(t) for t in rng.integers(0, vocab, size=n)]


#: worst relative error seen per test (printed at the end of a run, so the margin under each tolerance is known)
WORST = {}


def rel_err(got, want):
    """max |got - want| / max |want| over whole arrays (numpy or torch)."""
    import os
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    err = float(np.abs(got - want).max() / max(np.abs(want).max(), 1e-30))
    test = os.environ.get("PYTEST_CURRENT_TEST", "").split(" ")[0]
    WORST[test] = max(WORST.get(test, 0.0), err)
    return err


#: tolerances on max|dlogit| / max|logit| against the float64 plain implementation
#: about twice the worst error any engine test shows (float32 1.5e-6, bfloat16 4.8e-3; the run prints them at its end)
TOL = {"float32": 4e-6, "bfloat16": 1e-2}
