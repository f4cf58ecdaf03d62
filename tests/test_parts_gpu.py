"""Each part of a layer alone, built through its registry with its sizes as parameters, against the
plain implementation's function for that part; long decoding; the first tokens of a sequence; a
far key that stands out."""
import math

import numpy as np
import pytest
import torch

import plain_llama as P
from helpers import TINY, TOL, make_model_dir, random_tokens, rel_err

pytestmark = pytest.mark.gpu


def _rand(shape, std, seed, dtype):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * std).to(dtype)


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-6), (torch.bfloat16, 2 ** -8)])
def test_rmsnorm_part(dtype, tol):
    from fastgguf_b200.parts import run_part
    w = (1 + _rand((72,), 0.1, 1, torch.float32)).to(dtype)
    x = _rand((5, 72), 2.0, 2, torch.float32)
    got = run_part("norm", "rmsnorm", dict(size=72, eps=3e-4), {"weight": w}, dtype, x=x.numpy())
    want = P.plain_rmsnorm(x.double(), w.double(), 3e-4)
    assert (torch.from_numpy(got).double() - want).abs().max() <= tol * want.abs().max()


def test_rotary_tables_follow_the_plain_angles():
    from fastgguf_b200.parts import position_tables
    scaling = {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
               "original_max_position_embeddings": 8192}
    cos, sin, perm = position_tables("rope", dict(head_dim=64, theta=500000.0, scaling=scaling), 9000)
    assert perm == list(range(64))                      # halves layout over the whole head: rows stay where they are
    div = P.plain_rope_divisors({"rope_theta": 500000.0, "rope_scaling": scaling}, 64)
    for pos in (0, 1, 777, 8999):
        for j in (0, 5, 17, 31):
            ang = pos / (500000.0 ** (2.0 * j / 64)) / div[j]
            assert abs(cos[pos, j] - math.cos(ang)) < 1e-6 and abs(sin[pos, j] - math.sin(ang)) < 1e-6


def test_rotary_layouts_and_partial_rotation_become_row_permutations():
    """Adjacent pairs (the reference's own Llama layout, fastgguf.c:3138-3139) and a rotary dimension smaller than the
    head are brought to the kernels' pairs (j, j + head_dim/2) by a permutation of the q/k rows and identity entries."""
    from fastgguf_b200.parts import position_tables
    cos, sin, perm = position_tables("rope", dict(head_dim=8, theta=100.0, scaling=None, layout="adjacent"), 16)
    assert perm == [0, 2, 4, 6, 1, 3, 5, 7]
    assert abs(cos[3, 1] - math.cos(3 / 100.0 ** (2 / 8))) < 1e-6
    cos, sin, perm = position_tables("rope", dict(head_dim=8, theta=100.0, scaling=None, rotary_dim=4), 16)
    assert perm == [0, 1, 4, 5, 2, 3, 6, 7]             # rotated pairs (0,2), (1,3); dims 4..7 untouched
    assert abs(cos[5, 1] - math.cos(5 / 100.0 ** (2 / 4))) < 1e-6 and (cos[:, 2:] == 1).all() and (sin[:, 2:] == 0).all()
    cos, sin, perm = position_tables("rope", dict(head_dim=8, theta=100.0, scaling=None, rotary_dim=4, layout="adjacent"), 4)
    assert perm == [0, 2, 4, 5, 1, 3, 6, 7]


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 2e-2)])
@pytest.mark.parametrize("E,F", [(40, 56), (128, 320)])
def test_swiglu_part(E, F, dtype, tol):
    from fastgguf_b200.parts import run_part
    shapes = {"gate_proj.weight": (F, E), "up_proj.weight": (F, E), "down_proj.weight": (E, F)}
    W = {n: _rand(s, 0.2, i, dtype) for i, (n, s) in enumerate(shapes.items())}
    xn = _rand((9, E), 1.0, 7, dtype)
    res = _rand((9, E), 1.0, 8, torch.float32)
    out = run_part("feed_forward", "swiglu", dict(hidden_size=E, d_ff=F), W, dtype, x=xn.float().numpy(), residual=res.numpy())
    want = res.double() + P.plain_swiglu(xn.double(), W["gate_proj.weight"].double(), W["up_proj.weight"].double(),
                                         W["down_proj.weight"].double())
    assert rel_err(out, want) < tol


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 2e-2)])
def test_embedding_and_head_parts(dtype, tol):
    from fastgguf_b200.parts import run_part
    V, E = 77, 40
    table = _rand((V, E), 1.0, 3, dtype)
    toks = [5, 76, 0, 5]
    got = run_part("embedding", "embedding", dict(vocab_size=V, hidden_size=E), {"weight": table}, dtype, tokens=toks, out_cols=E)
    assert np.array_equal(got, table.float().numpy()[toks])
    got = run_part("embedding", "embedding", dict(vocab_size=V, hidden_size=E, scale=2.5), {"weight": table}, dtype, tokens=toks,
                   out_cols=E)
    assert np.allclose(got, 2.5 * table.float().numpy()[toks], rtol=1e-6)
    xn = _rand((6, E), 1.0, 4, dtype)
    got = run_part("head", "lm_head", dict(vocab_size=V, hidden_size=E), {"weight": table}, dtype, x=xn.float().numpy(), out_cols=V)
    assert rel_err(got, xn.double() @ table.double().T) < tol


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", ["b", "c"])
def test_attention_part_and_block_in_two_steps(tmp_path, which, dtype):
    """One layer's mixer and whole block, fed a sequence in two steps through a real cache."""
    from fastgguf_b200.engine.api import Engine
    cfg_dict, seed = TINY[which]
    model_dir = make_model_dir(tmp_path, cfg_dict, seed, torch.bfloat16)
    cfg, W = P.read_model_folder(model_dir)
    engine = Engine.from_dir(model_dir, dtype=dtype, max_tokens=512, max_batch=2)
    E = cfg["hidden_size"]
    T = 90
    x = _rand((T, E), 1.0, 5, torch.float32)
    Wd = {k: v.double() for k, v in W.items()}
    want_block = P.plain_layer(x.double(), Wd, "model.layers.1.", cfg, list(range(T)))
    slot = engine.acquire()
    got = []
    for lo, hi in ((0, 67), (67, T)):
        xs = np.ascontiguousarray(x[lo:hi].numpy())
        engine.block_forward(1, [(slot, hi - lo)], xs)
        got.append(torch.from_numpy(xs))
    assert engine.cache.length(slot) == T
    assert rel_err(torch.cat(got), want_block) < (1e-5 if dtype == "float32" else 2e-2)
    engine.release(slot)


def test_adjacent_pair_layout_equals_the_halves_layout_on_permuted_rows(tmp_path):
    """A model whose q/k rows are stored for adjacent rotary pairs gives the logits of the same model stored for halves
    pairs: the layout is a parameter of the position part, and the attention mixer permutes its rows at load."""
    from fastgguf_b200.engine.api import Engine
    from fastgguf_b200.engine.batch import StepEntry
    from fastgguf_b200.registry import config_from_dict, spec_from_config
    cfg_dict, seed = TINY["b"]
    model_dir = make_model_dir(tmp_path, cfg_dict, seed, torch.float32)
    cfg, W = P.read_model_folder(model_dir)
    H, KV, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    spec = spec_from_config(config_from_dict(cfg_dict))
    adj = {k: v.clone() for k, v in W.items()}
    for layer in spec.layers:
        layer.mixer.params["position"].params["layout"] = "adjacent"
    inv = [0] * hd                                       # stored row of halves index i: pairs (j, j + hd/2) -> (2j, 2j + 1)
    for j in range(hd // 2):
        inv[2 * j], inv[2 * j + 1] = j, j + hd // 2
    for i in range(cfg["num_hidden_layers"]):
        for n, heads in (("q", H), ("k", KV)):
            name = f"model.layers.{i}.self_attn.{n}_proj.weight"
            adj[name] = W[name].reshape(heads, hd, -1)[:, inv, :].reshape(heads * hd, -1)
    toks = random_tokens(50, cfg["vocab_size"], 3)
    want = P.plain_forward(cfg, W, toks).numpy()
    engine = Engine.from_spec(spec, adj, dtype="float32", max_tokens=256, max_batch=1)
    slot = engine.acquire()
    got = engine.step([StepEntry(slot, toks, list(range(50)))]).cpu().numpy()
    assert rel_err(got, want) < TOL["float32"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", ["a", "c"])
def test_long_decoding_and_first_tokens(tmp_path, which, dtype):
    """A sequence fed one token at a time from its very first token, across several pages."""
    from fastgguf_b200.engine.api import Engine
    from fastgguf_b200.engine.batch import StepEntry
    cfg_dict, seed = TINY[which]
    model_dir = make_model_dir(tmp_path, cfg_dict, seed, torch.bfloat16)
    cfg, W = P.read_model_folder(model_dir)
    toks = random_tokens(200, cfg["vocab_size"], 31)
    want = P.plain_forward(cfg, W, toks).numpy()
    engine = Engine.from_dir(model_dir, dtype=dtype, max_tokens=256, max_batch=1)
    slot = engine.acquire()
    rows = [engine.step([StepEntry(slot, [t], [0])]).cpu().numpy()[0] for t in toks]
    got = np.stack(rows)
    assert rel_err(got[:3], want[:3]) < TOL[dtype]                  # the first tokens of a sequence
    assert rel_err(got, want) < TOL[dtype]
    engine.release(slot)
    engine.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_far_key_that_stands_out(tmp_path, dtype):
    """Queries and keys of one layer are scaled up so that attention concentrates on single far keys:
    a key that is skipped, doubled or read from the wrong page then changes the logits visibly."""
    from fastgguf_b200.engine.api import Engine
    from fastgguf_b200.engine.batch import StepEntry
    import os
    cfg_dict, seed = TINY["c"]
    model_dir = make_model_dir(tmp_path, cfg_dict, seed, torch.bfloat16)
    path = os.path.join(model_dir, "model.safetensors")
    tensors = P.read_safetensors(path)
    for n in ("q_proj", "k_proj"):
        tensors[f"model.layers.0.self_attn.{n}.weight"] = (tensors[f"model.layers.0.self_attn.{n}.weight"].float() * 7).to(torch.bfloat16)
    P.write_safetensors(path, tensors)
    cfg, W = P.read_model_folder(model_dir)
    toks = random_tokens(450, cfg["vocab_size"], 41)
    want = P.plain_forward(cfg, W, toks).numpy()
    engine = Engine.from_dir(model_dir, dtype=dtype, max_tokens=1024, max_batch=2)
    slot = engine.acquire()
    head = engine.step([StepEntry(slot, toks[:400], list(range(400)))]).cpu().numpy()
    tail = [engine.step([StepEntry(slot, [t], [0])]).cpu().numpy()[0] for t in toks[400:]]
    got = np.concatenate([head, np.stack(tail)])
    # attention sharpened sevenfold amplifies the rounding of q and k: 1.1e-2 measured in bfloat16, 1.5e-6 in float32
    assert rel_err(got, want) < 2.5 * TOL[dtype]
