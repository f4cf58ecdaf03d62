"""Trace replay: the same requests whole, with the last 32 tokens one by one, and in batches of
unequal lengths (one batch after another so that slots and pages are used again), in 32-bit and
in bfloat16, all against the plain implementation."""
import numpy as np
import pytest
import torch

import plain_llama
from helpers import TINY, TOL, make_model_dir, random_tokens
from trace_tools import batched_trace, collect, run_trace, tail_trace, whole_trace

pytestmark = pytest.mark.gpu

LENGTHS = [5, 9, 1, 17, 3, 40, 11, 70, 33, 130]


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for which, (cfg_dict, seed) in TINY.items():
        d = make_model_dir(tmp_path_factory.mktemp(f"tiny_{which}"), cfg_dict, seed, torch.bfloat16)
        cfg, W = plain_llama.read_model_folder(d)
        requests = {f"r{i}": random_tokens(n, cfg["vocab_size"], 100 + i) for i, n in enumerate(LENGTHS)}
        want = {rid: plain_llama.plain_forward(cfg, W, toks).numpy() for rid, toks in requests.items()}
        out[which] = (d, cfg, requests, want)
    return out


def _compare(rows, want, requests, tol, what):
    assert len(rows) == sum(len(t) for t in requests.values()), what
    worst = 0.0
    for (rid, pos), row in rows.items():
        scale = np.abs(want[rid]).max()
        worst = max(worst, float(np.abs(row - want[rid][pos]).max() / scale))
    import os
    from helpers import WORST
    test = os.environ.get("PYTEST_CURRENT_TEST", "").split(" ")[0]
    WORST[test] = max(WORST.get(test, 0.0), worst)
    assert worst < tol, (what, worst)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", ["a", "b", "c", "d"])
def test_replay_three_cuts(tmp_path, models, which, dtype):
    model_dir, cfg, requests, want = models[which]
    V = cfg["vocab_size"]
    # whole: one live request at a time, so one request's pages are enough
    steps, index = whole_trace(requests)
    run_trace(model_dir, dtype, steps, str(tmp_path / "whole"), max_tokens=192)
    whole = collect(str(tmp_path / "whole"), steps, index, V)
    _compare(whole, want, requests, TOL[dtype], "whole")
    # the last 32 tokens one by one
    steps, index = tail_trace(requests, 32)
    run_trace(model_dir, dtype, steps, str(tmp_path / "tail"), max_tokens=192)
    tail = collect(str(tmp_path / "tail"), steps, index, V)
    _compare(tail, want, requests, TOL[dtype], "tail")
    # batches of 4 unequal requests, one after another; the cache holds just one batch
    steps, index = batched_trace(requests, 4)
    need = max(sum((len(requests[r]) + 63) // 64 * 64 for r in list(requests)[b:b + 4]) for b in range(0, 10, 4))
    run_trace(model_dir, dtype, steps, str(tmp_path / "batched"), max_tokens=need)
    batched = collect(str(tmp_path / "batched"), steps, index, V)
    _compare(batched, want, requests, TOL[dtype], "batched")
    # the cuts agree with one another much more closely than with the oracle in 32-bit
    if dtype == "float32":
        for key in whole:
            assert np.abs(whole[key] - tail[key]).max() < 1e-5
            assert np.abs(whole[key] - batched[key]).max() < 1e-5
