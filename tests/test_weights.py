"""Weights: the safetensors container, loading by name with one error, dtype policy, random folders.
Everything here runs on the host (the C++ reader and checker behind ``fastgguf_b200.weights``); the files
are written and read back by the test's own small safetensors code in ``plain_llama``."""
import json
import os
import struct

import pytest
import torch

import plain_llama
from helpers import TINY_A, TINY_B, make_model_dir


def _config(cfg_dict):
    from fastgguf_b200.registry import config_from_dict
    return config_from_dict(cfg_dict)


def _random_tensors(tmp_path, cfg_dict, seed):
    d = make_model_dir(tmp_path / f"src{seed}", cfg_dict, seed)
    return plain_llama.read_safetensors(os.path.join(d, "model.safetensors"))


def test_folder_tensors_reads_what_was_written(tmp_path):
    from fastgguf_b200.weights import folder_tensors
    t = {"a": torch.randn(3, 5).to(torch.bfloat16), "b.c": torch.arange(7, dtype=torch.int32),
         "d": torch.randn(2, 2, 2), "e": torch.zeros(0, 4)}
    plain_llama.write_safetensors(str(tmp_path / "model.safetensors"), t)
    got = {e["name"]: e for e in folder_tensors(str(tmp_path))}
    assert sorted(got) == sorted(t)
    assert got["a"] == {"name": "a", "dtype": "bfloat16", "shape": [3, 5]}
    assert got["b.c"]["dtype"] == "int32" and got["d"]["shape"] == [2, 2, 2] and got["e"]["shape"] == [0, 4]


def test_container_errors(tmp_path):
    from fastgguf_b200.weights import SafetensorsError, folder_tensors
    p = str(tmp_path / "model.safetensors")
    with pytest.raises(SafetensorsError, match="neither model.safetensors"):
        folder_tensors(str(tmp_path))
    open(p, "wb").write(b"abc")
    with pytest.raises(SafetensorsError, match="too short"):
        folder_tensors(str(tmp_path))
    open(p, "wb").write(struct.pack("<Q", 1000) + b"{}")
    with pytest.raises(SafetensorsError, match="header length"):
        folder_tensors(str(tmp_path))
    open(p, "wb").write(struct.pack("<Q", 5) + b"{nope")
    with pytest.raises(SafetensorsError, match="not valid JSON"):
        folder_tensors(str(tmp_path))

    def with_header(h, data=b"\0" * 8):
        blob = json.dumps(h).encode()
        open(p, "wb").write(struct.pack("<Q", len(blob)) + blob + data)

    with_header({"w": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]}})
    with pytest.raises(SafetensorsError, match="extends past the end"):
        folder_tensors(str(tmp_path))
    with_header({"w": {"dtype": "Q4_K", "shape": [2], "data_offsets": [0, 8]}})
    with pytest.raises(SafetensorsError, match="unsupported type Q4_K"):
        folder_tensors(str(tmp_path))
    with_header({"w": {"dtype": "F32", "shape": [3], "data_offsets": [0, 8]}})
    with pytest.raises(SafetensorsError, match="needs 12 bytes"):
        folder_tensors(str(tmp_path))
    with_header({"w": {"dtype": "F32"}})
    with pytest.raises(SafetensorsError, match="malformed"):
        folder_tensors(str(tmp_path))


def test_shards_and_a_tensor_in_two_of_them(tmp_path):
    from fastgguf_b200.weights import SafetensorsError, folder_tensors
    plain_llama.write_safetensors(str(tmp_path / "s1.safetensors"), {"a": torch.zeros(2), "b": torch.zeros(3)})
    plain_llama.write_safetensors(str(tmp_path / "s2.safetensors"), {"c": torch.zeros(4)})
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps(
        {"weight_map": {"a": "s1.safetensors", "b": "s1.safetensors", "c": "s2.safetensors"}}))
    assert [e["name"] for e in folder_tensors(str(tmp_path))] == ["a", "b", "c"]
    plain_llama.write_safetensors(str(tmp_path / "s2.safetensors"), {"c": torch.zeros(4), "a": torch.zeros(2)})
    with pytest.raises(SafetensorsError, match="is also in"):
        folder_tensors(str(tmp_path))
    (tmp_path / "model.safetensors.index.json").write_text("{}")
    with pytest.raises(SafetensorsError, match="not a shard index"):
        folder_tensors(str(tmp_path))


def test_one_error_lists_missing_unexpected_and_wrong(tmp_path):
    from fastgguf_b200.weights import WeightError, check_weights
    cfg = _config(TINY_B)
    t = _random_tensors(tmp_path, TINY_B, 1)
    del t["model.layers.1.mlp.up_proj.weight"], t["model.norm.weight"]
    t["model.layers.0.self_attn.q_proj.bias"] = torch.zeros(144)
    t["model.layers.2.self_attn.k_proj.weight"] = torch.zeros(48, 144, dtype=torch.bfloat16)
    t["model.embed_tokens.weight"] = torch.zeros(509, 144, dtype=torch.int32)
    plain_llama.write_safetensors(str(tmp_path / "model.safetensors"), t)
    for kwargs in (dict(model_dir=str(tmp_path)), dict(tensors=t)):           # a folder, and tensors in memory
        with pytest.raises(WeightError) as e:
            check_weights(cfg, **kwargs)
        err = e.value
        assert err.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
        assert err.unexpected == ["model.layers.0.self_attn.q_proj.bias"]
        assert len(err.wrong) == 2 and "[48, 144]" in str(err) and "[24, 144]" in str(err)
        for name in err.missing + err.unexpected:
            assert name in str(err)


def test_dtype_policy(tmp_path):
    """16-bit tensors become bfloat16, a tensor stored in 32 bits stays so; float32 engines widen all."""
    from fastgguf_b200.weights import check_weights
    cfg = _config(TINY_A)
    t = _random_tensors(tmp_path, TINY_A, 0)
    t["model.norm.weight"] = t["model.norm.weight"].float()
    t["model.layers.0.mlp.down_proj.weight"] = t["model.layers.0.mlp.down_proj.weight"].to(torch.float16)
    plain_llama.write_safetensors(str(tmp_path / "model.safetensors"), t)
    got = check_weights(cfg, model_dir=str(tmp_path), dtype="bfloat16")
    assert got["model.norm.weight"] == "float32"
    assert got["model.layers.0.mlp.down_proj.weight"] == "bfloat16"
    assert got["model.embed_tokens.weight"] == "bfloat16"
    wide = check_weights(cfg, model_dir=str(tmp_path), dtype="float32")
    assert set(wide.values()) == {"float32"}


def test_tied_head_ignores_a_stored_lm_head_and_untied_needs_it(tmp_path):
    from fastgguf_b200.weights import WeightError, check_weights, expected_tensors
    cfg = _config(TINY_A)
    t = _random_tensors(tmp_path, TINY_A, 0)
    assert "lm_head.weight" not in t and "lm_head.weight" not in expected_tensors(cfg)
    t["lm_head.weight"] = torch.zeros(256, 64, dtype=torch.bfloat16)
    plain_llama.write_safetensors(str(tmp_path / "model.safetensors"), t)
    check_weights(cfg, model_dir=str(tmp_path))
    # untied: the same file loads, and the head is the stored tensor
    untied = _config(dict(TINY_A, tie_word_embeddings=False))
    assert "lm_head.weight" in check_weights(untied, model_dir=str(tmp_path))
    del t["lm_head.weight"]
    plain_llama.write_safetensors(str(tmp_path / "model.safetensors"), t)
    with pytest.raises(WeightError) as e:
        check_weights(untied, model_dir=str(tmp_path))
    assert e.value.missing == ["lm_head.weight"]


def test_random_model_folder_is_deterministic(tmp_path):
    a = make_model_dir(tmp_path / "a", TINY_B, 5)
    b = make_model_dir(tmp_path / "b", TINY_B, 5)
    c = make_model_dir(tmp_path / "c", TINY_B, 6)
    fa, fb, fc = (plain_llama.read_safetensors(os.path.join(d, "model.safetensors")) for d in (a, b, c))
    assert sorted(fa) == sorted(fb)
    assert all(torch.equal(fa[n], fb[n]) for n in fa)
    assert not torch.equal(fa["lm_head.weight"], fc["lm_head.weight"])
    # a tensor's values depend on (seed, its name) alone: two tensors of one folder differ
    assert not torch.equal(fa["model.layers.0.mlp.up_proj.weight"], fa["model.layers.1.mlp.up_proj.weight"])
    cfg = json.load(open(os.path.join(a, "config.json")))
    assert cfg["architectures"] == ["LlamaForCausalLM"] and cfg["hidden_size"] == 144 and cfg["torch_dtype"] == "bfloat16"
    w = fa["model.layers.0.mlp.up_proj.weight"].float()
    n = fa["model.norm.weight"].float()
    assert abs(w.std().item() - 0.02) < 0.002 and abs(w.mean().item()) < 0.001
    assert abs(n.mean().item() - 1.0) < 0.01 and 0.005 < n.std().item() < 0.02
    # float32 folders hold the values the bfloat16 ones were rounded from
    f32 = plain_llama.read_safetensors(os.path.join(make_model_dir(tmp_path / "f", TINY_B, 5, "float32"), "model.safetensors"))
    assert f32["lm_head.weight"].dtype == torch.float32
    assert torch.equal(f32["lm_head.weight"].to(torch.bfloat16), fa["lm_head.weight"])
