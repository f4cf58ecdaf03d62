"""Generation through the entry point: greedy and sampled, graph-replayed and plain, against the
plain implementation; stop tokens, sequences that end earlier, batches one after another."""
import numpy as np
import pytest
import torch

import plain_llama
from helpers import TINY, make_model_dir, random_tokens

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for which, (cfg_dict, seed) in TINY.items():
        d = make_model_dir(tmp_path_factory.mktemp(f"gen_{which}"), cfg_dict, seed, torch.bfloat16)
        out[which] = (d,) + plain_llama.read_model_folder(d)
    return out


@pytest.mark.parametrize("use_graphs", [False, True])
@pytest.mark.parametrize("which,lens", [("a", [5, 9, 1]), ("b", [17, 3, 40, 11])])
def test_greedy_float32_matches_plain(models, which, lens, use_graphs):
    from fastgguf_b200.engine.api import Engine
    model_dir, cfg, W = models[which]
    prompts = [random_tokens(n, cfg["vocab_size"], 50 + i) for i, n in enumerate(lens)]
    engine = Engine.from_dir(model_dir, dtype="float32", max_tokens=1024, max_batch=4, use_graphs=use_graphs)
    out = engine.generate(prompts, temp=0, max_tokens=8, ignore_eos=True)
    for p, c in zip(prompts, out):
        want = plain_llama.plain_generate(cfg, W, p, max_tokens=8, temp=0, top_k=0, top_p=1.0, repeat_penalty=1.0,
                                          repeat_last_n=64)
        assert c.tokens == want and c.finish_reason == "length"
    engine.cache.check()
    assert engine.cache.live_slots() == []


@pytest.mark.parametrize("use_graphs", [False, True])
def test_sampled_float32_matches_plain(models, use_graphs):
    """Temperature 0.8 with the reference's default top-k / top-p, and a repeat penalty: same logits,
    same generator state, same token - also for the second batch, whose slots were used before."""
    from fastgguf_b200.engine.api import Engine
    from fastgguf_b200.sampling import request_seed
    model_dir, cfg, W = models["b"]
    prompts = [random_tokens(n, cfg["vocab_size"], 60 + i) for i, n in enumerate([17, 3, 40, 11, 6])]
    engine = Engine.from_dir(model_dir, dtype="float32", max_tokens=1024, max_batch=4, use_graphs=use_graphs)
    opts = dict(temp=0.8, top_k=64, top_p=0.95, repeat_penalty=1.3, repeat_last_n=16)
    out = engine.generate(prompts, max_tokens=12, seed=7, ignore_eos=True, batch_size=3, **opts)
    for i, (p, c) in enumerate(zip(prompts, out)):
        want = plain_llama.plain_generate(cfg, W, p, max_tokens=12, seed=request_seed(7, i), **opts)
        assert c.tokens == want, i


@pytest.mark.parametrize("use_graphs", [False, True])
def test_stop_tokens_and_early_finish(models, use_graphs):
    """A stop token ends its sequence without being emitted; the others go on; slots come back."""
    from fastgguf_b200.engine.api import Engine
    model_dir, cfg, W = models["a"]
    prompts = [random_tokens(n, cfg["vocab_size"], 70 + i) for i, n in enumerate([4, 12, 7, 2, 9])]
    free = [plain_llama.plain_generate(cfg, W, p, max_tokens=10, temp=0, top_k=0, top_p=1.0, repeat_penalty=1.0,
                                       repeat_last_n=64) for p in prompts]
    stops = {free[0][3], free[2][0]}               # sequence 0 stops before its 4th token, sequence 2 at once
    want = []
    for toks in free:
        cut = next((k for k, t in enumerate(toks) if t in stops), None)
        want.append((toks if cut is None else toks[:cut], "length" if cut is None else "stop"))
    engine = Engine.from_dir(model_dir, dtype="float32", max_tokens=512, max_batch=2, use_graphs=use_graphs)
    out = engine.generate(prompts, temp=0, max_tokens=10, stop_ids=sorted(stops), batch_size=2)
    assert [(c.tokens, c.finish_reason) for c in out] == want
    engine.cache.check()
    assert engine.cache.live_slots() == []


def test_greedy_bfloat16_is_plausible(models):
    """bfloat16 greedy tokens: each chosen token's float64 logit lies within rounding of the maximum."""
    from fastgguf_b200.engine.api import Engine
    model_dir, cfg, W = models["b"]
    prompts = [random_tokens(n, cfg["vocab_size"], 80 + i) for i, n in enumerate([20, 5, 33])]
    engine = Engine.from_dir(model_dir, dtype="bfloat16", max_tokens=1024, max_batch=4)
    out = engine.generate(prompts, temp=0, max_tokens=16, ignore_eos=True)
    for p, c in zip(prompts, out):
        assert len(c.tokens) == 16
        logits = plain_llama.plain_forward(cfg, W, p + c.tokens).numpy()
        for k, tok in enumerate(c.tokens):
            row = logits[len(p) - 1 + k]
            assert row[tok] >= row.max() - 3e-2 * np.abs(row).max()


def test_context_full_ends_with_length(models):
    from fastgguf_b200.engine.api import Engine
    model_dir, cfg, W = models["a"]
    engine = Engine.from_dir(model_dir, dtype="float32", max_tokens=256, max_batch=2, max_seq_len=64)
    out = engine.generate([random_tokens(60, cfg["vocab_size"], 90)], temp=0, max_tokens=0, ignore_eos=True)
    # 60 prompt tokens + 4 fed tokens fill the 64 positions; the 5th sampled token is still emitted
    assert len(out[0].tokens) == 5 and out[0].finish_reason == "length"


def test_calls_that_differ_only_in_seed_share_one_backend_and_few_option_sets_are_kept(models):
    """The recorded decode graphs belong to a set of sampling options, not to a seed: new seeds record nothing, and of
    many option sets only the most recent few keep their graphs and activation memory."""
    from fastgguf_b200.engine.api import Engine
    d, cfg, _ = models["a"]
    engine = Engine.from_dir(d, dtype="bfloat16", max_tokens=1024, max_batch=2)
    prompts = [[3, 5, 7, 11], [2, 4]]
    engine.generate(prompts, max_tokens=4, temp=0.9, top_k=8, top_p=0.9, seed=1, ignore_eos=True)
    first = engine.stats()
    assert first["backends"] == 1 and first["graphs"] >= 1
    outs = [engine.generate(prompts, max_tokens=4, temp=0.9, top_k=8, top_p=0.9, seed=s, ignore_eos=True) for s in (2, 3, 2)]
    after = engine.stats()
    assert after["backends"] == 1 and after["graphs"] == first["graphs"]
    assert [c.tokens for c in outs[0]] == [c.tokens for c in outs[2]]          # the seed still decides the tokens
    for i in range(6):
        engine.generate(prompts, max_tokens=2, temp=0.5 + 0.1 * i, top_k=8, top_p=0.9, seed=1, ignore_eos=True)
    assert engine.stats()["backends"] <= 4


def test_profile_lists_launchers_and_records_no_graph(models):
    from fastgguf_b200.engine.api import Engine
    d, cfg, W = models["b"]
    engine = Engine.from_dir(d, dtype="bfloat16", max_tokens=1024, max_batch=2)
    prompts = [[3, 5, 7, 11, 13], [2, 4]]
    plain = engine.generate(prompts, max_tokens=5, temp=0, ignore_eos=True, use_graphs=False)
    engine.profile(True)
    out = engine.generate(prompts, max_tokens=5, temp=0, ignore_eos=True)
    rows = engine.profile_report()
    engine.profile(False)
    assert [c.tokens for c in out] == [c.tokens for c in plain]              # eager steps: the same tokens
    names = {r["name"].split(" ")[0] for r in rows}
    assert rows and all(r["calls"] > 0 and r["ms"] > 0 for r in rows)
    assert "fg_gemm_tc" in names or "fg_gemm_generic" in names
    assert any(n.startswith("fg_attention") or n.startswith("fg_rope") for n in names)
    assert rows == sorted(rows, key=lambda r: -r["ms"])
    assert engine.profile_report() == []                                       # a report clears the records


def test_plain_kernels_switch_gives_the_same_tokens(models, monkeypatch):
    """FASTGGUF_PLAIN_KERNELS=1 puts a bfloat16 engine on the any-size kernels: the same results up to rounding."""
    from fastgguf_b200.engine.api import Engine
    from fastgguf_b200.engine.batch import StepEntry
    d, cfg, W = models["a"]
    toks = random_tokens(40, cfg["vocab_size"], 9)
    fast = Engine.from_dir(d, dtype="bfloat16", max_tokens=256, max_batch=1)
    monkeypatch.setenv("FASTGGUF_PLAIN_KERNELS", "1")
    slow = Engine.from_dir(d, dtype="bfloat16", max_tokens=256, max_batch=1)
    monkeypatch.delenv("FASTGGUF_PLAIN_KERNELS")
    got = []
    for e in (fast, slow):
        e.profile(True)
        s = e.acquire()
        got.append(np.asarray(e.step_host([StepEntry(s, toks, list(range(len(toks))))])))
        e.release(s)
        names = {r["name"].split(" ")[0] for r in e.profile_report()}
        e.profile(False)
        assert ("fg_gemm_tc" in names) == (e is fast) and ("fg_gemm_generic" in names) == (e is slow)
    want = plain_llama.plain_forward(cfg, W, toks).numpy()
    scale = np.abs(want).max()
    assert np.abs(got[1] - want).max() <= 1e-2 * scale and np.abs(got[0] - want).max() <= 1e-2 * scale
