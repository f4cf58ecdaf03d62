"""A context beyond 16K positions through the engine itself: one ~17,000-token prompt (the tcgen05 prefill attention
over hundreds of pages), then decode steps that take more than 8 splits of the pages - the scratch-memory path and the
merge kernel - in bfloat16, against the plain parts at the last positions.  The model has ONE layer, so the plain side
needs attention only for the rows it compares; queries and keys are scaled up so that attention concentrates on single
far keys, and a split that is dropped, doubled or merged wrongly changes the logits visibly."""
import math
import os

import numpy as np
import pytest
import torch

import plain_llama as P
from helpers import TINY_C, make_model_dir, random_tokens, rel_err

pytestmark = pytest.mark.gpu


def _plain_rows(cfg, W, toks, rows):
    """Logits of a one-layer model at ``rows`` (float64): keys and values of every position, attention for the rows."""
    W = {k: v.double() for k, v in W.items()}
    E, H, KV, hd = P.sizes(cfg)
    T, p = len(toks), "model.layers.0."
    x = P.plain_embedding(W["model.embed_tokens.weight"], toks)
    n1 = P.plain_rmsnorm(x, W[p + "input_layernorm.weight"], cfg["rms_norm_eps"])
    div = P.plain_rope_divisors(cfg, hd)
    pos = list(range(T))
    k = P.plain_rope((n1 @ W[p + "self_attn.k_proj.weight"].T).reshape(T, KV, hd), pos, cfg["rope_theta"], div)
    v = (n1 @ W[p + "self_attn.v_proj.weight"].T).reshape(T, KV, hd)
    q = P.plain_rope((n1[rows] @ W[p + "self_attn.q_proj.weight"].T).reshape(len(rows), H, hd), rows, cfg["rope_theta"], div)
    out = []
    for i, r in enumerate(rows):
        heads = []
        for h in range(H):
            kv = h // (H // KV)
            w = torch.softmax((k[:r + 1, kv] @ q[i, h]) / math.sqrt(hd), 0)
            heads.append(w @ v[:r + 1, kv])
        h1 = torch.cat(heads) @ W[p + "self_attn.o_proj.weight"].T + x[r]
        n2 = P.plain_rmsnorm(h1[None], W[p + "post_attention_layernorm.weight"], cfg["rms_norm_eps"])
        h2 = P.plain_swiglu(n2, W[p + "mlp.gate_proj.weight"], W[p + "mlp.up_proj.weight"], W[p + "mlp.down_proj.weight"])[0] + h1
        xf = P.plain_rmsnorm(h2[None], W["model.norm.weight"], cfg["rms_norm_eps"])[0]
        out.append(xf @ W["model.embed_tokens.weight"].T)
    return torch.stack(out).numpy()


def test_a_context_of_seventeen_thousand_positions(tmp_path):
    from fastgguf_b200.engine.api import Engine
    from fastgguf_b200.engine.batch import StepEntry
    cfg_dict = dict(TINY_C, num_hidden_layers=1, max_position_embeddings=20480)
    model_dir = make_model_dir(tmp_path, cfg_dict, 7, "bfloat16")
    path = os.path.join(model_dir, "model.safetensors")
    tensors = P.read_safetensors(path)
    for n in ("q_proj", "k_proj"):
        name = f"model.layers.0.self_attn.{n}.weight"
        tensors[name] = (tensors[name].float() * 6).to(torch.bfloat16)
    P.write_safetensors(path, tensors)
    cfg, W = P.read_model_folder(model_dir)
    T, extra = 17000, 3
    toks = random_tokens(T + extra, cfg["vocab_size"], 17)
    rows = [T - 1, T, T + 1, T + 2]
    want = _plain_rows(cfg, W, toks, rows)
    engine = Engine.from_dir(model_dir, dtype="bfloat16", max_tokens=17472, max_batch=1)
    slot = engine.acquire()
    got = [engine.step([StepEntry(slot, toks[:T], [T - 1])]).cpu().numpy()[0]]
    for t in toks[T:]:
        got.append(engine.step([StepEntry(slot, [t], [0])]).cpu().numpy()[0])       # 266 pages: more than 8 splits, scratch + merge
    assert rel_err(np.stack(got), want) < 3e-2
    engine.check_device()
    engine.release(slot)
    engine.cache.check()
