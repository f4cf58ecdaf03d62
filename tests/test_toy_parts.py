"""Generality of the layer parts, shown with toy parts defined HERE (``tests/toy_parts.cu``, compiled by this test into
a library of its own) and registered through the C interface without touching the framework's files: a mixer with
fixed-size state of its own (no keys, no values), a feed-forward with routing, another position encoding, a scaled
embedding and another block arrangement; a schedule that runs a layer twice (two caches) and an entry that reads
another entry's cache; a windowed cache group.  The toy models are stepped whole, in pieces and in unequal batches,
and GENERATED from through the entry point (recorded decode steps on and off, batches one after another so that slots
and their state rows are used again, a request that stops early), all against a plain computation."""
import math
import os
import subprocess

import numpy as np
import pytest
import torch

import plain_llama as P

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
E, H, KV, HD, F, V = 48, 3, 1, 16, 80, 101


@pytest.fixture(scope="module")
def toys(tmp_path_factory):
    """Compile the toy library and register its kinds (once per process)."""
    from fastgguf_b200.csrc.build import _nvcc
    from fastgguf_b200.parts import register_part_library
    out = str(tmp_path_factory.mktemp("toys") / "libtoy_parts.so")
    cmd = [_nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-O2", "-std=c++17", "-Xcompiler", "-fPIC", "-shared",
           "-I", os.path.join(ROOT, "fastgguf_b200", "csrc"), "-o", out, os.path.join(ROOT, "tests", "toy_parts.cu")]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    return register_part_library(out, {("mixer", "toy_running_mean"): "toy_running_mean_vtable",
                                       ("feed_forward", "toy_routed"): "toy_routed_vtable",
                                       ("position", "toy_half_rotary"): "toy_half_rotary_vtable",
                                       ("embedding", "toy_scaled_embed"): "toy_scaled_embed_vtable",
                                       ("block", "toy_parallel"): "toy_parallel_vtable"})


def _weights(spec, seed, dtype):
    """Random tensors for a spec from what its parts declare, scaled up so that the parts matter."""
    from fastgguf_b200.weights import expected_tensors
    g = torch.Generator().manual_seed(seed)
    W = {}
    for name, d in sorted(expected_tensors(spec).items()):
        t = torch.randn(d["shape"], generator=g) * d["std"]
        W[name] = (1 + t if d["init"] == "one_plus_normal" else 5 * t).to(dtype)
    return W


def _spec():
    from fastgguf_b200.engine.spec import LayerSpec, ModelSpec, PartSpec, RunSpec
    rope = PartSpec("rope", dict(head_dim=HD, theta=10000.0, scaling=None))
    norm = lambda name: PartSpec("rmsnorm", dict(size=E, eps=1e-5), {"weight": name})
    ffn = lambda p: PartSpec("swiglu", dict(hidden_size=E, d_ff=F), {f"{n}_proj.weight": f"{p}.ffn.{n}" for n in ("gate", "up", "down")})
    attn = PartSpec("gqa_attention", dict(hidden_size=E, n_heads=H, n_kv_heads=KV, head_dim=HD, position=rope),
                    {f"{n}_proj.weight": f"l0.attn.{n}" for n in "qkvo"})
    toy = PartSpec("toy_running_mean", dict(hidden_size=E), {"mix.weight": "l1.mix"})
    layers = [LayerSpec("prenorm", attn, ffn("l0"), norm("l0.n1"), norm("l0.n2")),
              LayerSpec("prenorm", toy, ffn("l1"), norm("l1.n1"), norm("l1.n2"))]
    # attention layer, toy layer, the attention layer AGAIN (its own cache), and once more reading entry 0's cache
    schedule = [RunSpec(0), RunSpec(1), RunSpec(0), RunSpec(0, cache_from=0)]
    return ModelSpec(hidden_size=E, vocab_size=V, max_positions=512,
                     embedding=PartSpec("embedding", dict(vocab_size=V, hidden_size=E), {"weight": "emb"}),
                     layers=layers, schedule=schedule, final_norm=norm("nf"),
                     head=PartSpec("lm_head", dict(vocab_size=V, hidden_size=E), {"weight": "emb"}))


def _plain(W, toks):
    """The toy model on a whole sequence, from the plain implementation's parts."""
    W = {k: v.double() for k, v in W.items()}
    T = len(toks)
    x = P.plain_embedding(W["emb"], toks)
    pos = list(range(T))

    def attention_layer(x, shared_kv=None):
        n1 = P.plain_rmsnorm(x, W["l0.n1"], 1e-5)
        q = P.plain_rope((n1 @ W["l0.attn.q"].T).reshape(T, H, HD), pos, 10000.0, [1.0] * (HD // 2))
        if shared_kv is None:
            k = P.plain_rope((n1 @ W["l0.attn.k"].T).reshape(T, KV, HD), pos, 10000.0, [1.0] * (HD // 2))
            v = (n1 @ W["l0.attn.v"].T).reshape(T, KV, HD)
        else:
            k, v = shared_kv
        h1 = P.plain_attention(q, k, v, 1 / math.sqrt(HD)).reshape(T, H * HD) @ W["l0.attn.o"].T + x
        n2 = P.plain_rmsnorm(h1, W["l0.n2"], 1e-5)
        return P.plain_swiglu(n2, W["l0.ffn.gate"], W["l0.ffn.up"], W["l0.ffn.down"]) + h1, (k, v)

    x, kv0 = attention_layer(x)
    n1 = P.plain_rmsnorm(x, W["l1.n1"], 1e-5)
    means = n1.cumsum(0) / torch.arange(1, T + 1, dtype=torch.float64)[:, None]
    h1 = means @ W["l1.mix"].T + x
    x = P.plain_swiglu(P.plain_rmsnorm(h1, W["l1.n2"], 1e-5), W["l1.ffn.gate"], W["l1.ffn.up"], W["l1.ffn.down"]) + h1
    x, _ = attention_layer(x)
    x, _ = attention_layer(x, shared_kv=kv0)
    return (P.plain_rmsnorm(x, W["nf"], 1e-5) @ W["emb"].T).numpy()


def _err(got, w):
    return float(np.abs(got - w).max() / np.abs(w).max())


@pytest.mark.parametrize("dtype,tol", [("float32", 2e-5), ("bfloat16", 3e-2)])
def test_toy_mixer_with_state_and_a_schedule_with_repeats(toys, dtype, tol):
    from fastgguf_b200.engine.api import Engine
    from fastgguf_b200.engine.batch import StepEntry
    from fastgguf_b200.weights import expected_tensors
    spec = _spec()
    expected = expected_tensors(spec)
    assert "l1.mix" in expected and len(expected) == 17            # the repeated layer's tensors appear once
    W = _weights(spec, 9, torch.bfloat16)
    engine = Engine.from_spec(spec, W, dtype=dtype, max_tokens=512, max_batch=3)
    info = engine.info()
    assert len(info["groups"]) == 1 and info["groups"][0]["entries"] == [0, 2]   # entry 3 borrows, entry 1 keeps no keys
    assert info["state_bytes"] == (3 + 1) * ((E + 1) * 4 + 12)     # one row per slot plus the spare, rounded to 16 bytes
    Wf = {k: v.float() for k, v in W.items()}
    rng = np.random.default_rng(0)
    seqs = [rng.integers(0, V, size=n).tolist() for n in (70, 5, 33)]
    want = [_plain(Wf, s) for s in seqs]
    # whole, each alone
    for s, w in zip(seqs, want):
        slot = engine.acquire()
        got = engine.step([StepEntry(slot, s, list(range(len(s))))]).cpu().numpy()
        engine.release(slot)
        assert _err(got, w) < tol
    # an unequal batch: prompts (a prefix of each) in one step, then one token each; shorter ones end earlier
    slots = [engine.acquire() for _ in seqs]                       # slots used before: their state was zeroed again
    heads = [max(1, len(s) // 2) for s in seqs]
    out = engine.step([StepEntry(sl, s[:h], list(range(h))) for sl, s, h in zip(slots, seqs, heads)]).cpu().numpy()
    got = [[r for r in out[sum(heads[:i]):sum(heads[:i + 1])]] for i in range(3)]
    fed = list(heads)
    while any(f < len(s) for f, s in zip(fed, seqs)):
        live = [i for i in range(3) if fed[i] < len(seqs[i])]
        out = engine.step([StepEntry(slots[i], [seqs[i][fed[i]]], [0]) for i in live]).cpu().numpy()
        for r, i in zip(out, live):
            got[i].append(r)
            fed[i] += 1
    for g, w in zip(got, want):
        assert _err(np.stack(g), w) < tol
    for sl in slots:
        engine.release(sl)
    engine.cache.check()


def _plain_greedy(plain, W, prompt, max_tokens, stop=()):
    """A plain loop over a whole-sequence function: the reference's loop (fastgguf.c:5284-5309) for one sequence."""
    toks, out = list(prompt), []
    for _ in range(max_tokens):
        nxt = int(np.argmax(plain(W, toks)[-1]))
        if nxt in stop:
            return out, "stop"
        out.append(nxt)
        toks.append(nxt)
    return out, "length"


@pytest.mark.parametrize("use_graphs", [False, True])
def test_generation_with_a_state_mixer_borrowed_caches_and_repeats(toys, use_graphs):
    """Generation through the entry point with the running-mean mixer (state rows per slot), the repeated layer and the
    borrowed cache: two slots for five requests, so slots and their state rows are used again; one request stops early."""
    from fastgguf_b200.engine.api import Engine
    spec = _spec()
    W = _weights(spec, 11, torch.float32)
    engine = Engine.from_spec(spec, W, dtype="float32", max_tokens=512, max_batch=2, use_graphs=use_graphs)
    rng = np.random.default_rng(5)
    prompts = [rng.integers(0, V, size=n).tolist() for n in (9, 70, 3, 64, 21)]
    free = [_plain_greedy(_plain, W, p, 7)[0] for p in prompts]
    stops = {free[1][2]}                                          # request 1 stops before its third token
    want = [_plain_greedy(_plain, W, p, 7, stops) for p in prompts]
    out = engine.generate(prompts, temp=0, max_tokens=7, stop_ids=sorted(stops), batch_size=2)
    assert [(c.tokens, c.finish_reason) for c in out] == want
    assert engine.cache.live_slots() == []
    engine.cache.check()


# ------------------------------------------------------------------------------------------------
# another position encoding, a feed-forward with routing, a scaled embedding and another block arrangement

def _spec2(block="prenorm", embed_scale=None):
    from fastgguf_b200.engine.spec import LayerSpec, ModelSpec, PartSpec, RunSpec
    pos = PartSpec("toy_half_rotary", dict(head_dim=HD, theta=100.0, rot=5, scale=0.5))
    norm = lambda name: PartSpec("rmsnorm", dict(size=E, eps=1e-6), {"weight": name})
    attn = PartSpec("gqa_attention", dict(hidden_size=E, n_heads=H, n_kv_heads=KV, head_dim=HD, position=pos, window=40),
                    {f"{n}_proj.weight": f"a.{n}" for n in "qkvo"})
    names = {"router.weight": "r.w"}
    for e in range(2):
        names[f"experts.{e}.up"] = f"r.{e}.up"
        names[f"experts.{e}.down"] = f"r.{e}.down"
    routed = PartSpec("toy_routed", dict(hidden_size=E, d_ff=F), names)
    layers = [LayerSpec(block, attn, routed, norm("n1"), norm("n2"))]
    if embed_scale is None:
        emb = PartSpec("embedding", dict(vocab_size=V, hidden_size=E), {"weight": "emb"})
    else:
        emb = PartSpec("toy_scaled_embed", dict(vocab_size=V, hidden_size=E, scale=embed_scale), {"weight": "emb"})
    return ModelSpec(hidden_size=E, vocab_size=V, max_positions=512, embedding=emb,
                     layers=layers, schedule=[RunSpec(0)], final_norm=norm("nf"),
                     head=PartSpec("lm_head", dict(vocab_size=V, hidden_size=E), {"weight": "head"}))


def _plain2(W, toks, parallel=False, embed_scale=1.0):
    W = {k: v.double() for k, v in W.items()}
    T = len(toks)
    x = P.plain_embedding(W["emb"], toks) * embed_scale
    n1 = P.plain_rmsnorm(x, W["n1"], 1e-6)
    # half rotary: a divisor of 1 / scale on the rotated pairs, "infinite" on the others (angle 0)
    div = [2.0] * 5 + [1e300] * (HD // 2 - 5)
    pos = list(range(T))
    q = P.plain_rope((n1 @ W["a.q"].T).reshape(T, H, HD), pos, 100.0, div)
    k = P.plain_rope((n1 @ W["a.k"].T).reshape(T, KV, HD), pos, 100.0, div)
    v = (n1 @ W["a.v"].T).reshape(T, KV, HD)
    h1 = P.plain_attention(q, k, v, 1 / math.sqrt(HD), window=40).reshape(T, H * HD) @ W["a.o"].T + x
    n2 = P.plain_rmsnorm(x if parallel else h1, W["n2"], 1e-6)       # a parallel block normalises its INPUT twice
    pick = (n2 @ W["r.w"].T).argmax(-1)
    out = h1.clone()
    for t in range(T):
        e = int(pick[t])
        out[t] += torch.relu(n2[t] @ W[f"r.{e}.up"].T) @ W[f"r.{e}.down"].T
    return (P.plain_rmsnorm(out, W["nf"], 1e-6) @ W["head"].T).numpy()


def test_toy_position_encoding_and_routed_feed_forward(toys):
    """float32, so that the router's choice is the plain computation's; windowed attention of the framework."""
    from fastgguf_b200.engine.api import Engine
    from fastgguf_b200.engine.batch import StepEntry
    spec = _spec2()
    W = _weights(spec, 4, torch.float32)
    engine = Engine.from_spec(spec, W, dtype="float32", max_tokens=512, max_batch=2)
    assert engine.info()["groups"][0]["window"] == 40
    rng = np.random.default_rng(1)
    toks = rng.integers(0, V, size=150).tolist()
    want = _plain2(W, toks)
    slot = engine.acquire()
    head = engine.step([StepEntry(slot, toks[:100], list(range(100)))]).cpu().numpy()
    tail = [engine.step([StepEntry(slot, [t], [0])]).cpu().numpy()[0] for t in toks[100:]]
    got = np.concatenate([head, np.stack(tail)])
    assert _err(got, want) < 5e-5
    # the windowed group gave pages back: 150 positions with a window of 40 keep at most two pages
    assert engine.cache.free_pages(0) >= 8 - 2
    engine.release(slot)
    engine.cache.check()


@pytest.mark.parametrize("use_graphs", [False, True])
def test_generation_with_a_windowed_group_a_scaled_embedding_and_a_parallel_block(toys, use_graphs):
    """The windowed group under generation: decoding runs past two page releases; the embedding kind (scale 3) and the
    block arrangement come from the test's library."""
    from fastgguf_b200.engine.api import Engine
    spec = _spec2(block="toy_parallel", embed_scale=3.0)
    W = _weights(spec, 6, torch.float32)
    plain = lambda W, t: _plain2(W, t, parallel=True, embed_scale=3.0)
    engine = Engine.from_spec(spec, W, dtype="float32", max_tokens=1024, max_batch=2, use_graphs=use_graphs)
    rng = np.random.default_rng(7)
    prompts = [rng.integers(0, V, size=n).tolist() for n in (30, 61, 5)]
    want = [_plain_greedy(plain, W, p, 140 if i == 0 else 6) for i, p in enumerate(prompts)]
    out = engine.generate(prompts[:1], temp=0, max_tokens=140, stop_ids=[])          # 30 + 140 positions: pages 0 and 1 leave
    out += engine.generate(prompts[1:], temp=0, max_tokens=6, stop_ids=[], batch_size=2)
    assert [(c.tokens, c.finish_reason) for c in out] == want
    engine.cache.check()


def test_bfloat16_windowed_decoding_under_recorded_steps(toys):
    """bfloat16 with head size 64, so that the tensor-core decode kernel reads the windowed group: recorded decode steps
    past two page releases (the device tables keep stale ids of pages that went back), against the plain implementation."""
    from fastgguf_b200.engine.api import Engine
    from fastgguf_b200.engine.spec import LayerSpec, ModelSpec, PartSpec, RunSpec
    E2, H2, KV2, HD2, F2 = 128, 4, 2, 64, 192
    rope = PartSpec("rope", dict(head_dim=HD2, theta=10000.0, scaling=None))
    norm = lambda name: PartSpec("rmsnorm", dict(size=E2, eps=1e-5), {"weight": name})
    attn = PartSpec("gqa_attention", dict(hidden_size=E2, n_heads=H2, n_kv_heads=KV2, head_dim=HD2, position=rope, window=64),
                    {f"{n}_proj.weight": f"a.{n}" for n in "qkvo"})
    ffn = PartSpec("swiglu", dict(hidden_size=E2, d_ff=F2), {f"{n}_proj.weight": f"f.{n}" for n in ("gate", "up", "down")})
    spec = ModelSpec(hidden_size=E2, vocab_size=V, max_positions=1024,
                     embedding=PartSpec("embedding", dict(vocab_size=V, hidden_size=E2), {"weight": "emb"}),
                     layers=[LayerSpec("prenorm", attn, ffn, norm("n1"), norm("n2"))], schedule=[RunSpec(0)],
                     final_norm=norm("nf"), head=PartSpec("lm_head", dict(vocab_size=V, hidden_size=E2), {"weight": "emb"}))
    W = _weights(spec, 8, torch.bfloat16)
    Wd = {k: v.double() for k, v in W.items()}

    def plain(toks):
        T = len(toks)
        x = P.plain_embedding(Wd["emb"], toks)
        n1 = P.plain_rmsnorm(x, Wd["n1"], 1e-5)
        pos, ones = list(range(T)), [1.0] * (HD2 // 2)
        q = P.plain_rope((n1 @ Wd["a.q"].T).reshape(T, H2, HD2), pos, 10000.0, ones)
        k = P.plain_rope((n1 @ Wd["a.k"].T).reshape(T, KV2, HD2), pos, 10000.0, ones)
        v = (n1 @ Wd["a.v"].T).reshape(T, KV2, HD2)
        h1 = P.plain_attention(q, k, v, 1 / math.sqrt(HD2), window=64).reshape(T, H2 * HD2) @ Wd["a.o"].T + x
        n2 = P.plain_rmsnorm(h1, Wd["n2"], 1e-5)
        out = P.plain_swiglu(n2, Wd["f.gate"], Wd["f.up"], Wd["f.down"]) + h1
        return (P.plain_rmsnorm(out, Wd["nf"], 1e-5) @ Wd["emb"].T).numpy()

    engine = Engine.from_spec(spec, W, dtype="bfloat16", max_tokens=1024, max_batch=2, use_graphs=True)
    rng = np.random.default_rng(9)
    prompts = [rng.integers(0, V, size=n).tolist() for n in (40, 100)]
    out = engine.generate(prompts, temp=0, max_tokens=150, stop_ids=[])
    for p, c in zip(prompts, out):
        assert len(c.tokens) == 150
        logits = plain(p + c.tokens)
        for k, tok in enumerate(c.tokens):
            row = logits[len(p) - 1 + k]
            assert row[tok] >= row.max() - 3e-2 * np.abs(row).max(), (k, tok)
    engine.cache.check()
