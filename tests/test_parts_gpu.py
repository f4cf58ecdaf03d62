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


def _runtime(dtype):
    from fastgguf_b200.parts.base import Runtime
    return Runtime(torch.device("cuda"), dtype)


def _rand(shape, std, seed, dtype):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * std).to(dtype)


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-6), (torch.bfloat16, 2 ** -8)])
def test_rmsnorm_part(dtype, tol):
    from fastgguf_b200.parts import lookup
    norm = lookup("norm", "rmsnorm")(_runtime(dtype), size=72, eps=3e-4)
    assert norm.tensor_specs()["weight"].shape == (72,)
    w = (1 + _rand((72,), 0.1, 1, torch.float32)).to(dtype)
    norm.load({"weight": w.cuda()})
    x = _rand((5, 72), 2.0, 2, torch.float32)
    want = P.plain_rmsnorm(x.double(), w.double(), 3e-4)
    assert (norm.forward(x.cuda()).cpu().double() - want).abs().max() <= tol * want.abs().max()


def test_rotary_tables_follow_the_plain_angles():
    from fastgguf_b200.parts import lookup
    scaling = {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
               "original_max_position_embeddings": 8192}
    rope = lookup("position", "rope")(_runtime(torch.bfloat16), head_dim=64, theta=500000.0, scaling=scaling)
    rope.prepare(9000)
    div = P.plain_rope_divisors({"rope_theta": 500000.0, "rope_scaling": scaling}, 64)
    for pos in (0, 1, 777, 8999):
        for j in (0, 5, 17, 31):
            ang = pos / (500000.0 ** (2.0 * j / 64)) / div[j]
            assert abs(rope.cos[pos, j].item() - math.cos(ang)) < 1e-6 and abs(rope.sin[pos, j].item() - math.sin(ang)) < 1e-6


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 2e-2)])
@pytest.mark.parametrize("E,F", [(40, 56), (128, 320)])
def test_swiglu_part(E, F, dtype, tol):
    from fastgguf_b200.parts import lookup
    ffn = lookup("feed_forward", "swiglu")(_runtime(dtype), hidden_size=E, d_ff=F)
    W = {n: _rand(s.shape, 0.2, i, dtype) for i, (n, s) in enumerate(ffn.tensor_specs().items())}
    ffn.load({k: v.cuda() for k, v in W.items()})
    xn = _rand((9, E), 1.0, 7, dtype)
    res = _rand((9, E), 1.0, 8, torch.float32)
    out = res.clone().cuda()
    ffn.forward(xn.cuda(), None, out)
    want = res.double() + P.plain_swiglu(xn.double(), W["gate_proj.weight"].double(), W["up_proj.weight"].double(),
                                         W["down_proj.weight"].double())
    assert rel_err(out.cpu(), want) < tol


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", ["b", "c"])
def test_attention_part_and_block_in_two_steps(tmp_path, which, dtype):
    """One layer's mixer and whole block, fed a sequence in two steps through a real cache."""
    from fastgguf_b200.engine.api import Engine
    from fastgguf_b200.engine.batch import StepEntry, build_batch
    cfg_dict, seed = TINY[which]
    model_dir = make_model_dir(tmp_path, cfg_dict, seed, torch.bfloat16)
    cfg, W = P.read_model_folder(model_dir)
    engine = Engine.from_dir(model_dir, dtype=dtype, max_tokens=512, max_batch=2)
    model, cache = engine.model, engine.cache
    E = cfg["hidden_size"]
    T = 90
    x = _rand((T, E), 1.0, 5, torch.float32)
    Wd = {k: v.double() for k, v in W.items()}
    want_block = P.plain_layer(x.double(), Wd, "model.layers.1.", cfg, list(range(T)))
    block, io = model.blocks[1], model._io[1]
    slot = engine.acquire()
    got = []
    for lo, hi in ((0, 67), (67, T)):
        entries = [StepEntry(slot, [0] * (hi - lo), [])]
        cache.reserve([(slot, hi - lo)])
        batch = build_batch(entries, cache, engine.device)
        xs = x[lo:hi].clone().cuda()
        block.forward(xs, batch, io)
        cache.commit([(slot, hi - lo)])
        got.append(xs.cpu())
    assert rel_err(torch.cat(got), want_block) < (1e-5 if dtype == "float32" else 2e-2)
    engine.release(slot)


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
    from fastgguf_b200.weights.safetensors_io import SafetensorsFile, write_safetensors
    import os
    cfg_dict, seed = TINY["c"]
    model_dir = make_model_dir(tmp_path, cfg_dict, seed, torch.bfloat16)
    path = os.path.join(model_dir, "model.safetensors")
    f = SafetensorsFile(path)
    tensors = {n: f.tensor(n).clone() for n in f.names()}
    for n in ("q_proj", "k_proj"):
        tensors[f"model.layers.0.self_attn.{n}.weight"] = (tensors[f"model.layers.0.self_attn.{n}.weight"].float() * 7).to(torch.bfloat16)
    write_safetensors(path, tensors)
    cfg, W = P.read_model_folder(model_dir)
    toks = random_tokens(450, cfg["vocab_size"], 41)
    want = P.plain_forward(cfg, W, toks).numpy()
    engine = Engine.from_dir(model_dir, dtype=dtype, max_tokens=1024, max_batch=2)
    slot = engine.acquire()
    head = engine.step([StepEntry(slot, toks[:400], list(range(400)))]).cpu().numpy()
    tail = [engine.step([StepEntry(slot, [t], [0])]).cpu().numpy()[0] for t in toks[400:]]
    got = np.concatenate([head, np.stack(tail)])
    assert rel_err(got, want) < TOL[dtype]
