"""One layer with the layer sizes of the large configurations (Llama 3.2 3B: 24 heads in groups of 3,
head size 128; Llama 3.1 8B: d_ff 14336), a small vocabulary, bfloat16: prompts of unequal lengths in
one step, then a few decoded tokens, against the plain implementation (float32 on the CPU)."""
import numpy as np
import pytest
import torch

import plain_llama
from helpers import TINY_B, make_model_dir, random_tokens, rel_err

pytestmark = pytest.mark.gpu

SHAPES = {
    "3b": dict(hidden_size=3072, num_attention_heads=24, num_key_value_heads=8, head_dim=128, intermediate_size=8192),
    "8b": dict(hidden_size=4096, num_attention_heads=32, num_key_value_heads=8, head_dim=128, intermediate_size=14336),
}


@pytest.mark.parametrize("which", ["3b", "8b"])
def test_one_layer_of_a_large_configuration(tmp_path, which):
    from fastgguf_b200.engine.api import Engine
    from fastgguf_b200.engine.batch import StepEntry
    cfg_dict = dict(TINY_B, num_hidden_layers=1, vocab_size=515, max_position_embeddings=4096, **SHAPES[which])
    cfg_dict["rope_scaling"] = dict(TINY_B["rope_scaling"], factor=8.0, original_max_position_embeddings=128)
    model_dir = make_model_dir(tmp_path, cfg_dict, 11, torch.bfloat16)
    cfg, W = plain_llama.read_model_folder(model_dir)
    lens, extra = [150, 3, 70], 4
    seqs = [random_tokens(n + extra, cfg["vocab_size"], 200 + i) for i, n in enumerate(lens)]
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
    from fastgguf_b200.ops import fast_attention, fast_gemm
    assert fast_gemm.pipeline_error() == 0 and fast_attention.prefill_tc_error() == 0


def test_many_prompt_steps_of_a_few_hundred_tokens_in_a_row(tmp_path):
    """Prompts of 129 to 400 tokens through two layers of the 1B layer sizes, 240 steps back to back without anything
    between them that waits for the device: the output and down projections run split along K here (partial products,
    then a kernel that adds them), and every kernel may start while the ones before it still run.  The same prompt
    gives the same bits at the start and at the end."""
    from fastgguf_b200.engine.api import Engine
    from fastgguf_b200.engine.batch import StepEntry
    from fastgguf_b200.ops import fast_gemm
    cfg_dict = dict(TINY_B, num_hidden_layers=2, vocab_size=515, max_position_embeddings=4096, hidden_size=2048,
                    num_attention_heads=32, num_key_value_heads=8, head_dim=64, intermediate_size=8192)
    cfg_dict["rope_scaling"] = dict(TINY_B["rope_scaling"], factor=8.0, original_max_position_embeddings=128)
    assert fast_gemm.workspace_bytes(200, 2048, 8192, fast_gemm.EPI_ADD_F32) > 0        # the split is taken at these sizes
    model_dir = make_model_dir(tmp_path, cfg_dict, 12, torch.bfloat16)
    engine = Engine.from_dir(model_dir, dtype="bfloat16", max_tokens=1024, max_batch=2)
    prompts = {n: random_tokens(n, cfg_dict["vocab_size"], 300 + n) for n in (129, 160, 192, 256, 300, 400)}
    first = {}
    for i in range(240):
        n = list(prompts)[i % len(prompts)]
        slot = engine.acquire()
        out = engine.step([StepEntry(slot, prompts[n], [n - 1])])
        engine.release(slot)
        if n not in first:
            first[n] = out.clone()
        elif i >= 234:
            assert torch.equal(out, first[n])
    torch.cuda.synchronize()
    assert fast_gemm.pipeline_error() == 0


def test_recorded_decode_steps_of_more_than_128_sequences(tmp_path):
    """136 sequences decode together: above 128 rows the projections of a step run on the prefill kernels, the output
    and down projections split along K, all of it inside the recorded step.  Recorded and eager steps give the same
    tokens."""
    from fastgguf_b200.engine.api import Engine
    cfg_dict = dict(TINY_B, num_hidden_layers=2, vocab_size=515, max_position_embeddings=4096, hidden_size=2048,
                    num_attention_heads=32, num_key_value_heads=8, head_dim=64, intermediate_size=8192)
    cfg_dict["rope_scaling"] = dict(TINY_B["rope_scaling"], factor=8.0, original_max_position_embeddings=128)
    model_dir = make_model_dir(tmp_path, cfg_dict, 13, torch.bfloat16)
    B = 136
    engine = Engine.from_dir(model_dir, dtype="bfloat16", max_tokens=B * 128, max_batch=B, max_seq_len=256)
    prompts = [random_tokens(3 + (7 * i) % 40, cfg_dict["vocab_size"], 500 + i) for i in range(B)]
    runs = [engine.generate(prompts, temp=0.0, max_tokens=12, ignore_eos=True, batch_size=B, use_graphs=g) for g in (True, False)]
    assert [c.tokens for c in runs[0]] == [c.tokens for c in runs[1]]
    assert all(len(c.tokens) == 12 for c in runs[0])
