"""Weights: the safetensors container, loading by name with one error, dtype policy, random folders."""
import json
import os
import struct

import pytest
import torch

from helpers import TINY_A, TINY_B, make_model_dir


def _expected(cfg_dict, dtype=torch.bfloat16):
    from fastgguf_b200.engine.model import DecoderModel
    from fastgguf_b200.parts.base import Runtime
    from fastgguf_b200.registry import config_from_dict, spec_from_config
    model = DecoderModel(spec_from_config(config_from_dict(cfg_dict)), Runtime(torch.device("cpu"), dtype))
    return model


def test_safetensors_round_trip(tmp_path):
    from fastgguf_b200.weights import SafetensorsFile, write_safetensors
    t = {"a": torch.randn(3, 5).to(torch.bfloat16), "b.c": torch.arange(7, dtype=torch.int32),
         "d": torch.randn(2, 2, 2), "e": torch.zeros(0, 4)}
    path = str(tmp_path / "x.safetensors")
    write_safetensors(path, t, {"k": "v"})
    f = SafetensorsFile(path)
    assert sorted(f.names()) == sorted(t) and f.metadata == {"k": "v"}
    for k, v in t.items():
        assert torch.equal(f.tensor(k), v) and f.tensor(k).dtype == v.dtype


def test_container_errors(tmp_path):
    from fastgguf_b200.weights import SafetensorsError, SafetensorsFile
    p = str(tmp_path / "m.safetensors")
    with pytest.raises(SafetensorsError, match="cannot open"):
        SafetensorsFile(p)
    open(p, "wb").write(b"abc")
    with pytest.raises(SafetensorsError, match="too short"):
        SafetensorsFile(p)
    open(p, "wb").write(struct.pack("<Q", 1000) + b"{}")
    with pytest.raises(SafetensorsError, match="header length"):
        SafetensorsFile(p)
    open(p, "wb").write(struct.pack("<Q", 5) + b"{nope")
    with pytest.raises(SafetensorsError, match="not valid JSON"):
        SafetensorsFile(p)

    def with_header(h, data=b"\0" * 8):
        blob = json.dumps(h).encode()
        open(p, "wb").write(struct.pack("<Q", len(blob)) + blob + data)
    with_header({"w": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]}})
    with pytest.raises(SafetensorsError, match="extends past the end"):
        SafetensorsFile(p)
    with_header({"w": {"dtype": "Q4_K", "shape": [2], "data_offsets": [0, 8]}})
    with pytest.raises(SafetensorsError, match="unsupported type Q4_K"):
        SafetensorsFile(p)
    with_header({"w": {"dtype": "F32", "shape": [3], "data_offsets": [0, 8]}})
    with pytest.raises(SafetensorsError, match="needs 12 bytes"):
        SafetensorsFile(p)
    with_header({"w": {"dtype": "F32"}})
    with pytest.raises(SafetensorsError, match="malformed"):
        SafetensorsFile(p)


def test_one_error_lists_missing_unexpected_and_wrong(tmp_path):
    from fastgguf_b200.weights import FolderSource, WeightError, load_tensors, random_tensors, write_safetensors
    from fastgguf_b200.registry import config_from_dict
    cfg = config_from_dict(TINY_B)
    model = _expected(TINY_B)
    t = random_tensors(cfg, 1)
    del t["model.layers.1.mlp.up_proj.weight"], t["model.norm.weight"]
    t["model.layers.0.self_attn.q_proj.bias"] = torch.zeros(144)
    t["model.layers.2.self_attn.k_proj.weight"] = torch.zeros(48, 144, dtype=torch.bfloat16)
    t["model.embed_tokens.weight"] = torch.zeros(509, 144, dtype=torch.int32)
    write_safetensors(str(tmp_path / "model.safetensors"), t)
    with pytest.raises(WeightError) as e:
        load_tensors(FolderSource(str(tmp_path)), model.expected_tensors(), torch.bfloat16, torch.device("cpu"))
    err = e.value
    assert err.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert err.unexpected == ["model.layers.0.self_attn.q_proj.bias"]
    assert len(err.wrong) == 2 and "[48, 144]" in str(err) and "[24, 144]" in str(err)
    for name in err.missing + err.unexpected:
        assert name in str(err)


def test_dtype_policy(tmp_path):
    """16-bit tensors become bfloat16, a tensor stored in 32 bits stays so; float32 engines widen all."""
    from fastgguf_b200.weights import FolderSource, load_tensors, random_tensors, write_safetensors
    from fastgguf_b200.registry import config_from_dict
    t = random_tensors(config_from_dict(TINY_A), 0)
    t["model.norm.weight"] = t["model.norm.weight"].float()
    t["model.layers.0.mlp.down_proj.weight"] = t["model.layers.0.mlp.down_proj.weight"].to(torch.float16)
    write_safetensors(str(tmp_path / "model.safetensors"), t)
    exp = _expected(TINY_A).expected_tensors()
    got = load_tensors(FolderSource(str(tmp_path)), exp, torch.bfloat16, torch.device("cpu"))
    assert got["model.norm.weight"].dtype == torch.float32
    assert got["model.layers.0.mlp.down_proj.weight"].dtype == torch.bfloat16
    assert got["model.embed_tokens.weight"].dtype == torch.bfloat16
    wide = load_tensors(FolderSource(str(tmp_path)), exp, torch.float32, torch.device("cpu"))
    assert all(v.dtype == torch.float32 for v in wide.values())
    assert torch.equal(wide["model.embed_tokens.weight"], t["model.embed_tokens.weight"].float())


def test_tied_head_ignores_a_stored_lm_head_and_untied_needs_it(tmp_path):
    from fastgguf_b200.weights import FolderSource, WeightError, load_tensors, random_tensors, write_safetensors
    from fastgguf_b200.registry import config_from_dict, spec_from_config
    cfg = config_from_dict(TINY_A)
    t = random_tensors(cfg, 0)
    assert "lm_head.weight" not in t
    t["lm_head.weight"] = torch.zeros(256, 64, dtype=torch.bfloat16)
    write_safetensors(str(tmp_path / "model.safetensors"), t)
    spec = spec_from_config(cfg)
    load_tensors(FolderSource(str(tmp_path)), _expected(TINY_A).expected_tensors(), torch.bfloat16,
                 torch.device("cpu"), spec.ignored_tensors)
    # untied: the same file loads, and the head is the stored tensor
    got = load_tensors(FolderSource(str(tmp_path)), _expected(dict(TINY_A, tie_word_embeddings=False)).expected_tensors(),
                       torch.bfloat16, torch.device("cpu"))
    assert "lm_head.weight" in got
    del t["lm_head.weight"]
    write_safetensors(str(tmp_path / "model.safetensors"), t)
    with pytest.raises(WeightError) as e:
        load_tensors(FolderSource(str(tmp_path)), _expected(dict(TINY_A, tie_word_embeddings=False)).expected_tensors(),
                     torch.bfloat16, torch.device("cpu"))
    assert e.value.missing == ["lm_head.weight"]


def test_random_model_folder_is_deterministic(tmp_path):
    from fastgguf_b200.weights import SafetensorsFile
    a = make_model_dir(tmp_path / "a", TINY_B, 5)
    b = make_model_dir(tmp_path / "b", TINY_B, 5)
    c = make_model_dir(tmp_path / "c", TINY_B, 6)
    fa, fb, fc = (SafetensorsFile(os.path.join(d, "model.safetensors")) for d in (a, b, c))
    assert sorted(fa.names()) == sorted(fb.names())
    assert all(torch.equal(fa.tensor(n), fb.tensor(n)) for n in fa.names())
    assert not torch.equal(fa.tensor("lm_head.weight"), fc.tensor("lm_head.weight"))
    cfg = json.load(open(os.path.join(a, "config.json")))
    assert cfg["architectures"] == ["LlamaForCausalLM"] and cfg["hidden_size"] == 144
    w = fa.tensor("model.layers.0.mlp.up_proj.weight").float()
    n = fa.tensor("model.norm.weight").float()
    assert abs(w.std().item() - 0.02) < 0.002 and abs(n.mean().item() - 1.0) < 0.01 and 0.005 < n.std().item() < 0.02


def test_missing_weight_file(tmp_path):
    from fastgguf_b200.weights import FolderSource, SafetensorsError
    with pytest.raises(SafetensorsError, match="neither model.safetensors"):
        FolderSource(str(tmp_path))
