"""The engine's C interface itself (``fg_config_from_json`` -> ``fg_engine_create`` -> ``fg_slot_acquire`` -> ``fg_step``),
called through its exported symbols without the Python classes: the three replay cuts on two tiny configurations in
32-bit and in bfloat16 against the plain implementation; status codes; and a C program that links the library."""
import ctypes
import json
import os
import subprocess
from ctypes import byref, c_int, c_void_p

import numpy as np
import pytest

import plain_llama
from helpers import TINY, TOL, make_model_dir, random_tokens
from trace_tools import batched_trace, tail_trace, whole_trace

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LENGTHS = [5, 9, 1, 17, 3, 40, 11, 70, 33]


def _create(model_dir, dtype, max_tokens, max_batch):
    from fastgguf_b200 import capi
    l = capi.lib()
    capi.ensure_kernel_libraries(capi.FG_BF16 if dtype == "bfloat16" else capi.FG_F32)
    cfg, eng = c_void_p(), c_void_p()
    assert l.fg_config_from_dir(model_dir.encode(), byref(cfg)) == 0, l.fg_last_error()
    opts = capi.EngineOptions()
    l.fg_engine_default_options(byref(opts))
    opts.dtype = capi.FG_BF16 if dtype == "bfloat16" else capi.FG_F32
    opts.max_tokens, opts.max_batch = max_tokens, max_batch
    assert l.fg_engine_create(cfg, model_dir.encode(), byref(opts), byref(eng)) == 0, l.fg_last_error()
    return l, cfg, eng


def _replay(l, eng, steps, index, V):
    """Feed a trace through fg_slot_acquire / fg_step / fg_slot_release; returns {(request, position): logits row}."""
    slot_of, rows = {}, {}
    for rec, idx in zip(steps, index):
        slots, n_tok, tokens, want, at = [], [], [], [], 0
        for e in rec["entries"]:
            if e["id"] not in slot_of:
                s = c_int()
                assert l.fg_slot_acquire(eng, byref(s)) == 0, l.fg_last_error()
                slot_of[e["id"]] = s.value
            slots.append(slot_of[e["id"]])
            n_tok.append(len(e["tokens"]))
            tokens.extend(e["tokens"])
            want.extend(at + w for w in e["want"])
            at += len(e["tokens"])
        out = np.zeros((len(want), V), dtype=np.float32)
        arr = lambda v: (c_int * max(1, len(v)))(*v)
        rc = l.fg_step(eng, len(slots), arr(slots), arr(n_tok), arr(tokens), len(want), arr(want), c_void_p(out.ctypes.data))
        assert rc == 0, l.fg_last_error()
        for key, row in zip(idx, out):
            rows[key] = row.copy()
        for rid in rec["end"]:
            assert l.fg_slot_release(eng, slot_of.pop(rid)) == 0
    assert l.fg_engine_cache_check(eng) == 0
    return rows


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", ["a", "b"])
def test_three_cuts_through_the_c_interface(tmp_path, which, dtype):
    cfg_dict, seed = TINY[which]
    model_dir = make_model_dir(tmp_path, cfg_dict, seed, "bfloat16")
    cfg, W = plain_llama.read_model_folder(model_dir)
    V = cfg["vocab_size"]
    requests = {f"r{i}": random_tokens(n, V, 300 + i) for i, n in enumerate(LENGTHS)}
    want = {rid: plain_llama.plain_forward(cfg, W, toks).numpy() for rid, toks in requests.items()}
    l, cfg_h, eng = _create(model_dir, dtype, max_tokens=256, max_batch=3)
    try:
        for name, (steps, index) in (("whole", whole_trace(requests)), ("tail", tail_trace(requests, 32)),
                                     ("batched", batched_trace(requests, 3))):
            rows = _replay(l, eng, steps, index, V)
            assert len(rows) == sum(len(t) for t in requests.values()), name
            worst = max(float(np.abs(row - want[rid][pos]).max() / np.abs(want[rid]).max()) for (rid, pos), row in rows.items())
            print(f"{which} {dtype} {name}: worst relative error {worst:.3g}")
            assert worst < TOL[dtype], (name, worst)
    finally:
        l.fg_engine_destroy(eng)
        l.fg_config_destroy(cfg_h)


def test_status_codes_of_the_engine(tmp_path):
    from fastgguf_b200 import capi
    cfg_dict, seed = TINY["a"]
    model_dir = make_model_dir(tmp_path, cfg_dict, seed, "bfloat16")
    l, cfg_h, eng = _create(model_dir, "float32", max_tokens=128, max_batch=2)
    arr = lambda v: (c_int * max(1, len(v)))(*v)
    out = np.zeros((1, 256), dtype=np.float32)
    ptr = c_void_p(out.ctypes.data)
    s0, s1, s2 = c_int(), c_int(), c_int()
    assert l.fg_slot_acquire(eng, byref(s0)) == 0 and l.fg_slot_acquire(eng, byref(s1)) == 0
    assert l.fg_slot_acquire(eng, byref(s2)) == capi.E_CAPACITY and b"slots" in l.fg_last_error()
    assert l.fg_step(eng, 1, arr([5]), arr([1]), arr([3]), 1, arr([0]), ptr) == capi.E_CACHE              # a slot nobody holds
    assert l.fg_step(eng, 1, arr([s0.value]), arr([1]), arr([256]), 1, arr([0]), ptr) == capi.E_TOKEN     # token outside the vocabulary
    assert b"outside the vocabulary" in l.fg_last_error()
    assert l.fg_step(eng, 1, arr([s0.value]), arr([0]), arr([3]), 0, None, None) == capi.E_TOKEN          # an empty step
    assert l.fg_step(eng, 1, arr([s0.value]), arr([1]), arr([3]), 1, arr([4]), ptr) == capi.E_TOKEN       # a wanted row out of range
    assert l.fg_step(eng, 2, arr([s0.value, s0.value]), arr([1, 1]), arr([3, 4]), 0, None, None) == capi.E_CACHE   # twice in one step
    assert l.fg_step(eng, 1, arr([s0.value]), arr([200]), arr([3] * 200), 0, None, None) == capi.E_CAPACITY
    n = c_int()
    assert l.fg_slot_length(eng, s0.value, byref(n)) == 0 and n.value == 0                               # nothing was changed
    assert l.fg_step(eng, 1, arr([s0.value]), arr([3]), arr([3, 4, 5]), 1, arr([2]), ptr) == 0
    assert l.fg_slot_length(eng, s0.value, byref(n)) == 0 and n.value == 3
    assert l.fg_slot_release(eng, s1.value) == 0 and l.fg_slot_release(eng, s1.value) == capi.E_CACHE
    assert l.fg_engine_cache_check(eng) == 0
    l.fg_engine_destroy(eng)
    # a folder whose weights do not fit: one error that lists everything
    W = plain_llama.read_safetensors(os.path.join(model_dir, "model.safetensors"))
    del W["model.norm.weight"]
    plain_llama.write_safetensors(os.path.join(model_dir, "model.safetensors"), W)
    opts = capi.EngineOptions()
    l.fg_engine_default_options(byref(opts))
    eng = c_void_p()
    assert l.fg_engine_create(cfg_h, model_dir.encode(), byref(opts), byref(eng)) == capi.E_WEIGHTS
    assert b"missing tensors (1): model.norm.weight" in l.fg_last_error()
    # a cache that cannot fit is refused by name before anything is allocated
    plain_llama.write_safetensors(os.path.join(model_dir, "model.safetensors"),
                                  plain_llama.read_safetensors(os.path.join(make_model_dir(tmp_path / "again", cfg_dict, seed), "model.safetensors")))
    opts.max_tokens = 1 << 31
    opts.dtype = capi.FG_F32
    assert l.fg_engine_create(cfg_h, model_dir.encode(), byref(opts), byref(eng)) == capi.E_DEVICE
    assert b"the cache does not fit" in l.fg_last_error()
    l.fg_config_destroy(cfg_h)


def test_a_c_program_generates(tmp_path):
    """tests/c_api_example.c links libfg_engine.so, generates 8 greedy tokens for 3 prompts; the same through Python."""
    from fastgguf_b200 import capi
    from fastgguf_b200.csrc.build import build_dir
    from fastgguf_b200.engine.api import Engine
    from fastgguf_b200.registry import config_from_dict
    capi.lib()
    capi.ensure_kernel_libraries(capi.FG_F32)
    exe = str(tmp_path / "example")
    lib_dir = build_dir()
    r = subprocess.run(["gcc", "-O1", "-o", exe, os.path.join(ROOT, "tests", "c_api_example.c"),
                        "-I", os.path.join(ROOT, "fastgguf_b200", "csrc"), "-L", lib_dir, "-lfg_engine", f"-Wl,-rpath,{lib_dir}"],
                       capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    r = subprocess.run([exe], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr
    got = [[int(t) for t in line.split()] for line in r.stdout.strip().splitlines()]
    assert len(got) == 3 and all(len(g) == 8 for g in got)
    src = open(os.path.join(ROOT, "tests", "c_api_example.c")).read()
    config = json.loads("".join(line.strip().strip('"').replace('\\"', '"') for line in src.split("CONFIG =")[1].split(";")[0].splitlines()))
    engine = Engine.from_random(config_from_dict(config), 7, dtype="float32", max_tokens=1024, max_batch=4)
    out = engine.generate([[5, 17, 3], [9], [200, 1, 1, 4, 77]], temp=0, max_tokens=8, stop_ids=[])
    assert [c.tokens for c in out] == got
