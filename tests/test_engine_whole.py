"""Each request alone and whole, through the engine's step function, against the plain implementation."""
import pytest
import torch

import plain_llama
from helpers import TINY, TOL, make_model_dir, random_tokens, rel_err

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", ["a", "b", "c", "d", "e"])
def test_whole_requests(tmp_path, which, dtype):
    from fastgguf_b200.engine.api import Engine
    from fastgguf_b200.engine.batch import StepEntry
    cfg_dict, seed = TINY[which]
    model_dir = make_model_dir(tmp_path, cfg_dict, seed, torch.bfloat16)
    cfg, W = plain_llama.read_model_folder(model_dir)
    engine = Engine.from_dir(model_dir, dtype=dtype, max_tokens=1024, max_batch=4)
    for n, s in ((1, 10), (7, 11), (70, 12), (200, 13)):
        toks = random_tokens(n, cfg["vocab_size"], s)
        want = plain_llama.plain_forward(cfg, W, toks).numpy()
        slot = engine.acquire()
        got = engine.step([StepEntry(slot, toks, list(range(n)))]).cpu().numpy()
        engine.release(slot)
        engine.cache.check()
        assert got.shape == want.shape
        assert rel_err(got, want) < TOL[dtype], (which, dtype, n)
