"""The command line: inspect / dump / random on the CPU, generate and selftest on the GPU."""
import json
import os
import subprocess
import sys

import pytest
import torch

from helpers import TINY_A, TINY_C, make_model_dir

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run(*args):
    return subprocess.run([sys.executable, "-m", "fastgguf_b200", *args], cwd=ROOT, capture_output=True, text=True)


def test_inspect_dump_random_and_usage(tmp_path):
    cfg_path = tmp_path / "cfg.json"
    cfg_path.write_text(json.dumps(TINY_A))
    p = run("random", str(cfg_path), str(tmp_path / "m"), "--seed", "4", "--dtype", "float32")
    assert p.returncode == 0 and os.path.exists(tmp_path / "m" / "model.safetensors")
    p = run("inspect", str(tmp_path / "m"))
    assert p.returncode == 0 and "LlamaForCausalLM" in p.stdout and "hidden_size = 64" in p.stdout
    assert "tensors: 20" in p.stdout and "model.embed_tokens.weight" in p.stdout
    p = run("inspect", str(tmp_path / "m"), "--json")
    assert json.loads(p.stdout)["config"]["q_dim"] == 64
    p = run("dump", str(tmp_path / "m"))
    assert p.returncode == 0 and "rope_theta = 10000.0" in p.stdout
    assert run("inspect", str(tmp_path / "nothing")).returncode == 2          # load errors exit 2
    p = run("generate", str(tmp_path / "m"), "--bogus", "1")
    assert p.returncode == 1 and "unknown option --bogus" in p.stdout        # usage errors exit 1
    assert run("frobnicate").returncode == 1


def test_generate_options_have_the_reference_names_and_defaults():
    from fastgguf_b200.cli import UsageError, parse_generate_args
    o = parse_generate_args([])
    assert (o["ctx"], o["temp"], o["top_k"], o["top_p"], o["repeat_penalty"], o["repeat_last_n"], o["max_tokens"]) == \
        (2048, 1.0, 64, 0.95, 1.0, 64, 512)
    o = parse_generate_args(["32", "--temp", "0", "--top-k", "0", "--seed", "9", "--prompt", "1,2 3", "--stop-id", "7",
                             "--stop-id", "11", "--ignore-eos"])
    assert o["ctx"] == 64                                   # at least 64, as the reference
    assert o["prompts"] == [[1, 2, 3]] and o["stop_ids"] == [7, 11] and o["ignore_eos"] and o["seed"] == 9
    assert not o["stream"] and parse_generate_args(["--stream"])["stream"]
    for bad in (["--temp"], ["--top-k", "x"], ["--stop-id", "eos"], ["--nope", "1"], ["abc"]):
        with pytest.raises(UsageError):
            parse_generate_args(bad)


@pytest.mark.gpu
def test_generate_command(tmp_path):
    d = make_model_dir(tmp_path, TINY_C, 2, torch.bfloat16)
    p = run("generate", d, "256", "--temp", "0", "--max-tokens", "6", "--prompt", "5,17,3", "--prompt", "9", "--json",
            "--ignore-eos")
    assert p.returncode == 0, p.stdout + p.stderr
    # with --json the standard output is the JSON document alone; the summary lines are on the standard error
    assert "[Sampler] greedy" in p.stderr and "[Config] LlamaForCausalLM: layers=2 embd=256 ctx=256" in p.stderr
    out = json.loads(p.stdout)
    assert [len(o["tokens"]) for o in out] == [6, 6] and all(o["finish_reason"] == "length" for o in out)
    t = run("generate", d, "256", "--temp", "0", "--max-tokens", "3", "--prompt", "5,17,3", "--ignore-eos")
    assert t.returncode == 0 and "[Sampler] greedy" in t.stdout and "[0] " in t.stdout and "[gen: 3 tok" in t.stdout
    q = run("generate", d, "256", "--temp", "0", "--max-tokens", "6", "--prompt", "5,17,3", "--prompt", "9", "--json",
            "--ignore-eos", "--dtype", "float32")
    assert q.returncode == 0


@pytest.mark.gpu
def test_selftest_command():
    p = run("selftest", "--quick")
    assert p.returncode == 0, p.stdout[-3000:] + p.stderr[-2000:]
    assert "ALL TESTS PASSED" in p.stdout and "FAIL " not in p.stdout
