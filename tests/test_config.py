"""Configuration: reading config.json keys, defaults, every validation error, the registry."""
import copy
import json

import pytest

from helpers import TINY_A, TINY_B


def test_reads_every_key_and_derives_sizes():
    from fastgguf_b200.registry import config_from_dict
    c = config_from_dict(TINY_B)
    assert (c.hidden_size, c.num_hidden_layers, c.num_attention_heads, c.num_key_value_heads) == (144, 3, 6, 1)
    assert (c.head_dim, c.intermediate_size, c.vocab_size) == (24, 384, 509)
    assert c.rms_norm_eps == 1e-6 and c.rope_theta == 500000.0
    assert c.rope_scaling.rope_type == "llama3" and c.rope_scaling.factor == 4.0
    assert c.rope_scaling.original_max_position_embeddings == 32
    assert c.eos_token_ids == (3, 5) and not c.tie_word_embeddings
    assert (c.q_dim, c.kv_dim, c.group_size) == (144, 24, 6)
    a = config_from_dict(TINY_A)
    assert a.rope_scaling.rope_type == "default" and a.tie_word_embeddings and a.eos_token_ids == (2,)
    # parameter count: layers * (qkv + o + 3 ffn + 2 norms) + embedding + final norm (+ head if untied)
    E, F, V = 64, 192, 256
    assert a.parameter_count() == 2 * (E * (64 + 2 * 32) + 64 * E + 3 * E * F + 2 * E) + V * E + E


def test_defaults_follow_the_reference():
    from fastgguf_b200.registry import config_from_dict
    d = {k: v for k, v in TINY_A.items() if k not in ("head_dim", "num_key_value_heads", "rms_norm_eps", "rope_theta")}
    c = config_from_dict(d)
    assert c.head_dim == 64 // 4 and c.num_key_value_heads == 4
    assert c.rms_norm_eps == 1e-6 and c.rope_theta == 10000.0


def test_round_trip_through_to_dict():
    from fastgguf_b200.registry import config_from_dict
    for d in (TINY_A, TINY_B):
        c = config_from_dict(d)
        assert config_from_dict(json.loads(json.dumps(c.to_dict()))) == c


def test_newer_key_spellings():
    from fastgguf_b200.registry import config_from_dict
    d = copy.deepcopy(TINY_B)
    rs = d.pop("rope_scaling")
    d["rope_parameters"] = dict(rs, rope_theta=d.pop("rope_theta"))
    d["dtype"] = "float32"
    c = config_from_dict(d)
    assert c.rope_theta == 500000.0 and c.rope_scaling.factor == 4.0 and c.torch_dtype == "float32"


@pytest.mark.parametrize("change,fragment", [
    ({"hidden_size": None}, "hidden_size"),
    ({"num_hidden_layers": 0}, "num_hidden_layers must be positive"),
    ({"num_key_value_heads": 3}, "multiple of"),
    ({"head_dim": 15}, "even"),
    ({"rms_norm_eps": 0.0}, "rms_norm_eps"),
    ({"rope_theta": -1.0}, "rope_theta"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"attention_bias": True}, "attention_bias"),
    ({"mlp_bias": True}, "mlp_bias"),
    ({"vocab_size": "many"}, "vocab_size"),
    ({"eos_token_id": 999}, "outside the vocabulary"),
    ({"eos_token_id": "x"}, "eos_token_id"),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 2.0}}, "yarn"),
    ({"rope_scaling": {"rope_type": "llama3", "factor": 2.0}}, "low_freq_factor"),
    ({"rope_scaling": {"rope_type": "llama3", "factor": 2.0, "low_freq_factor": 4.0, "high_freq_factor": 1.0,
                       "original_max_position_embeddings": 32}}, "high_freq_factor"),
])
def test_validation_errors_name_the_key(change, fragment):
    from fastgguf_b200.config import ConfigError
    from fastgguf_b200.registry import config_from_dict
    d = copy.deepcopy(TINY_A)
    for k, v in change.items():
        if v is None:
            d.pop(k)
        else:
            d[k] = v
    with pytest.raises(ConfigError) as e:
        config_from_dict(d)
    assert fragment in str(e.value)


def test_unknown_architecture_lists_registered_names():
    from fastgguf_b200.config import ConfigError
    from fastgguf_b200.registry import config_from_dict, registered_architectures
    assert "LlamaForCausalLM" in registered_architectures()
    with pytest.raises(ConfigError) as e:
        config_from_dict(dict(TINY_A, architectures=["MambaForCausalLM"]))
    assert "MambaForCausalLM" in str(e.value) and "LlamaForCausalLM" in str(e.value)
    with pytest.raises(ConfigError):
        config_from_dict({k: v for k, v in TINY_A.items() if k != "architectures"})


def test_config_json_errors(tmp_path):
    from fastgguf_b200.config import ConfigError
    from fastgguf_b200.registry import config_from_dir
    with pytest.raises(ConfigError, match="no such file"):
        config_from_dir(str(tmp_path))
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError, match="not valid JSON"):
        config_from_dir(str(tmp_path))


def test_spec_is_data_chosen_layer_by_layer():
    from fastgguf_b200.registry import config_from_dict, spec_from_config
    spec = spec_from_config(config_from_dict(TINY_B))
    assert len(spec.layers) == 3 and [r.layer for r in spec.schedule] == [0, 1, 2]
    assert spec.layers[1].mixer.kind == "gqa_attention" and spec.layers[1].feed_forward.kind == "swiglu"
    assert spec.layers[2].mixer.params["n_kv_heads"] == 1 and spec.layers[0].mixer_norm.params["eps"] == 1e-6
    assert spec.layers[2].mixer.tensors["q_proj.weight"] == "model.layers.2.self_attn.q_proj.weight"
    assert spec.head.tensors["weight"] == "lm_head.weight" and spec.stop_token_ids == (3, 5)
    tied = spec_from_config(config_from_dict(TINY_A))
    assert tied.head.tensors["weight"] == "model.embed_tokens.weight"


def test_cli_option_parsing_follows_the_reference():
    from fastgguf_b200.cli import UsageError, parse_generate_args
    o = parse_generate_args([])
    assert (o["ctx"], o["temp"], o["top_k"], o["top_p"], o["repeat_penalty"], o["repeat_last_n"], o["max_tokens"],
            o["seed"]) == (2048, 1.0, 64, 0.95, 1.0, 64, 512, 0)
    o = parse_generate_args(["32", "--temp", "0", "--top-k", "5", "--max-tokens", "7", "--seed", "9",
                             "--prompt", "1,2,3", "--prompt", "4 5"])
    assert o["ctx"] == 64 and o["temp"] == 0 and o["top_k"] == 5 and o["max_tokens"] == 7 and o["seed"] == 9
    assert o["prompts"] == [[1, 2, 3], [4, 5]]
    with pytest.raises(UsageError, match="unknown option"):
        parse_generate_args(["--bogus", "1"])
    with pytest.raises(UsageError, match="missing value"):
        parse_generate_args(["--temp"])


def test_stop_tokens_of_generation_config_are_added(tmp_path):
    """A folder's generation_config.json may name further end-of-turn tokens; the union is the stop set."""
    from fastgguf_b200.config.base import ConfigError
    from fastgguf_b200.registry import config_from_dir
    d = tmp_path / "m"
    d.mkdir()
    (d / "config.json").write_text(json.dumps(TINY_A))                     # eos_token_id 2
    assert config_from_dir(str(d)).eos_token_ids == (2,)                   # no second file: unchanged
    (d / "generation_config.json").write_text(json.dumps({"eos_token_id": [2, 7, 9], "temperature": 0.6}))
    assert config_from_dir(str(d)).eos_token_ids == (2, 7, 9)
    (d / "generation_config.json").write_text(json.dumps({"eos_token_id": 11}))
    assert config_from_dir(str(d)).eos_token_ids == (2, 11)
    (d / "generation_config.json").write_text(json.dumps({"do_sample": True}))
    assert config_from_dir(str(d)).eos_token_ids == (2,)
    (d / "generation_config.json").write_text(json.dumps({"eos_token_id": 100000}))
    with pytest.raises(ConfigError, match="outside the vocabulary"):
        config_from_dir(str(d))
    (d / "generation_config.json").write_text(json.dumps({"eos_token_id": "</s>"}))
    with pytest.raises(ConfigError, match="generation_config.json"):
        config_from_dir(str(d))
    (d / "generation_config.json").write_text("{not json")
    with pytest.raises(ConfigError, match="not valid JSON"):
        config_from_dir(str(d))
