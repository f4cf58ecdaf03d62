"""The dense Llama decoder as data: LlamaConfig -> ModelSpec.

Every layer is a pre-norm block of grouped-query attention with rotary encoding and a SwiGLU
feed-forward; the schedule runs the layers once, in order, each with a cache of its own.
Tensor names are those of a model folder's safetensors; the reference's GGUF names for the
same tensors are ``token_embd``, ``output``, ``output_norm``, ``blk.N.attn_norm``,
``blk.N.attn_{q,k,v,output}``, ``blk.N.ffn_norm``, ``blk.N.ffn_{gate,up,down}``
(fastgguf.c:4266-4278, :4292-4365).  The head is the embedding table again when
``tie_word_embeddings`` is set (the reference decides by the absence of ``output.weight``,
fastgguf.c:4269-4270).
"""
from __future__ import annotations

from ..config.llama import LlamaConfig
from ..engine.spec import LayerSpec, ModelSpec, PartSpec, RunSpec
from ..registry import register_architecture

#: tensors some checkpoints carry that the model does not use
IGNORED_TENSORS = (r"model\.layers\.\d+\.self_attn\.rotary_emb\.inv_freq",)


def build_spec(cfg: LlamaConfig) -> ModelSpec:
    E = cfg.hidden_size
    rope = PartSpec("rope", dict(head_dim=cfg.head_dim, theta=cfg.rope_theta, scaling=cfg.rope_scaling.to_dict()))
    layers = []
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        layers.append(LayerSpec(
            block="prenorm",
            mixer=PartSpec("gqa_attention",
                           dict(hidden_size=E, n_heads=cfg.num_attention_heads, n_kv_heads=cfg.num_key_value_heads,
                                head_dim=cfg.head_dim, position=rope),
                           {f"{n}_proj.weight": f"{p}self_attn.{n}_proj.weight" for n in "qkvo"}),
            feed_forward=PartSpec("swiglu", dict(hidden_size=E, d_ff=cfg.intermediate_size),
                                  {f"{n}_proj.weight": f"{p}mlp.{n}_proj.weight" for n in ("gate", "up", "down")}),
            mixer_norm=PartSpec("rmsnorm", dict(size=E, eps=cfg.rms_norm_eps),
                                {"weight": f"{p}input_layernorm.weight"}),
            feed_forward_norm=PartSpec("rmsnorm", dict(size=E, eps=cfg.rms_norm_eps),
                                       {"weight": f"{p}post_attention_layernorm.weight"}),
        ))
    head_name = "model.embed_tokens.weight" if cfg.tie_word_embeddings else "lm_head.weight"
    return ModelSpec(
        hidden_size=E, vocab_size=cfg.vocab_size, max_positions=cfg.max_position_embeddings,
        embedding=PartSpec("embedding", dict(vocab_size=cfg.vocab_size, hidden_size=E),
                           {"weight": "model.embed_tokens.weight"}),
        layers=layers,
        schedule=[RunSpec(i) for i in range(cfg.num_hidden_layers)],
        final_norm=PartSpec("rmsnorm", dict(size=E, eps=cfg.rms_norm_eps), {"weight": "model.norm.weight"}),
        head=PartSpec("lm_head", dict(vocab_size=cfg.vocab_size, hidden_size=E), {"weight": head_name}),
        stop_token_ids=tuple(cfg.eos_token_ids),
        ignored_tensors=IGNORED_TENSORS + ((r"lm_head\.weight",) if cfg.tie_word_embeddings else ()),
    )


register_architecture("LlamaForCausalLM", LlamaConfig, build_spec)
