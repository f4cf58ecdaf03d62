"""``LlamaConfig``: the dense Llama decoder's config.json.

The class is the Python name of the host's ``LlamaConfig`` (``csrc/host/config.hpp``): keys
hidden_size, num_hidden_layers, num_attention_heads, num_key_value_heads (default: heads), head_dim
(default: hidden / heads, fastgguf.c:4283), intermediate_size, vocab_size, rms_norm_eps (default 1e-6,
:4228), rope_theta (default 10000, :4224), rope_scaling (llama3 or none; also under
``rope_parameters``), max_position_embeddings, tie_word_embeddings, torch_dtype / dtype, bos_token_id,
eos_token_id (integer or list), hidden_act (silu), attention_bias / mlp_bias (must be false).
"""
from __future__ import annotations

from .base import ModelConfig


class LlamaConfig(ModelConfig):
    @classmethod
    def from_dict(cls, d: dict) -> "LlamaConfig":
        d = dict(d)
        d.setdefault("architectures", ["LlamaForCausalLM"])
        return super().from_dict(d)
