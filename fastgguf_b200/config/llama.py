"""``LlamaConfig``: the dense Llama decoder's config.json, typed.

Reference counterparts: the ``llama.*`` metadata keys read in ``model_load``
(fastgguf.c:4213-4229: block_count, embedding_length, rope.freq_base default 10000,
rope.dimension_count, attention.layer_norm_rms_epsilon default 1e-6), head_dim from
``attention.key_length`` else ``embedding_length / head_count`` (fastgguf.c:4281-4283), and
the divisibility checks on the projection shapes (fastgguf.c:4309-4314, 4330-4335).  The
llama3 frequency scaling has no code in the reference (GGUF files carry the finished divisors
as ``rope_freqs.weight``, fastgguf.c:4278, 3131); here the config carries its parameters and
``parts.rope`` computes the divisors.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import ClassVar, Optional

from .base import ConfigError, ModelConfig, take


@dataclass
class RopeScaling:
    """``rope_scaling`` of config.json.  ``rope_type`` is "default" (no scaling) or "llama3"."""

    rope_type: str = "default"
    factor: float = 1.0
    low_freq_factor: float = 1.0
    high_freq_factor: float = 1.0
    original_max_position_embeddings: int = 0

    @classmethod
    def from_dict(cls, d: Optional[dict]) -> "RopeScaling":
        if d is None:
            return cls()
        if not isinstance(d, dict):
            raise ConfigError("config.json: 'rope_scaling' must be an object or null")
        kind = d.get("rope_type", d.get("type", "default"))
        if kind in (None, "default"):
            return cls()
        if kind != "llama3":
            raise ConfigError(
                f"config.json: rope_scaling.rope_type '{kind}' is not supported (known: default, llama3)")
        w = "config.json rope_scaling"
        return cls(
            rope_type="llama3",
            factor=take(d, "factor", float, where=w),
            low_freq_factor=take(d, "low_freq_factor", float, where=w),
            high_freq_factor=take(d, "high_freq_factor", float, where=w),
            original_max_position_embeddings=take(d, "original_max_position_embeddings", int, where=w),
        )

    def to_dict(self) -> Optional[dict]:
        if self.rope_type == "default":
            return None
        return {
            "rope_type": self.rope_type,
            "factor": self.factor,
            "low_freq_factor": self.low_freq_factor,
            "high_freq_factor": self.high_freq_factor,
            "original_max_position_embeddings": self.original_max_position_embeddings,
        }


@dataclass
class LlamaConfig(ModelConfig):
    architecture_names: ClassVar[tuple] = ("LlamaForCausalLM",)

    hidden_size: int = 0
    num_hidden_layers: int = 0
    num_attention_heads: int = 0
    num_key_value_heads: int = 0
    head_dim: int = 0
    intermediate_size: int = 0
    vocab_size: int = 0
    rms_norm_eps: float = 0.0
    rope_theta: float = 0.0
    rope_scaling: RopeScaling = field(default_factory=RopeScaling)
    max_position_embeddings: int = 0
    tie_word_embeddings: bool = False
    torch_dtype: str = "bfloat16"
    bos_token_id: Optional[int] = None
    eos_token_ids: tuple = ()
    hidden_act: str = "silu"

    # ------------------------------------------------------------------ derived sizes
    @property
    def q_dim(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.num_key_value_heads * self.head_dim

    @property
    def group_size(self) -> int:
        return self.num_attention_heads // self.num_key_value_heads

    def parameter_count(self) -> int:
        E, F, V = self.hidden_size, self.intermediate_size, self.vocab_size
        per_layer = E * (self.q_dim + 2 * self.kv_dim) + self.q_dim * E + 3 * E * F + 2 * E
        head = 0 if self.tie_word_embeddings else V * E
        return self.num_hidden_layers * per_layer + V * E + E + head

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, d: dict) -> "LlamaConfig":
        H = take(d, "num_attention_heads", int)
        E = take(d, "hidden_size", int)
        # newer config files nest the rotary parameters under "rope_parameters"
        rp = d.get("rope_parameters") if isinstance(d.get("rope_parameters"), dict) else None
        theta_src = rp if (rp is not None and "rope_theta" in rp) else d
        scaling_src = d.get("rope_scaling")
        if scaling_src is None and rp is not None and rp.get("rope_type", "default") != "default":
            scaling_src = rp
        eos = d.get("eos_token_id")
        if eos is None:
            eos_ids: tuple = ()
        elif isinstance(eos, int) and not isinstance(eos, bool):
            eos_ids = (eos,)
        elif isinstance(eos, list) and all(isinstance(t, int) and not isinstance(t, bool) for t in eos):
            eos_ids = tuple(eos)
        else:
            raise ConfigError(f"config.json: 'eos_token_id' must be an integer or a list of integers, got {eos!r}")
        if take(d, "attention_bias", bool, False):
            raise ConfigError("config.json: attention_bias=true is not supported (the Llama path has no biases)")
        if take(d, "mlp_bias", bool, False):
            raise ConfigError("config.json: mlp_bias=true is not supported (the Llama path has no biases)")
        if H <= 0:
            raise ConfigError(f"config.json: num_attention_heads must be positive, got {H}")
        cfg = cls(
            hidden_size=E,
            num_hidden_layers=take(d, "num_hidden_layers", int),
            num_attention_heads=H,
            # absent: as many KV heads as heads (plain multi-head attention)
            num_key_value_heads=take(d, "num_key_value_heads", int, H),
            # absent: hidden_size / heads, the reference's fallback (fastgguf.c:4283)
            head_dim=take(d, "head_dim", int, E // H),
            intermediate_size=take(d, "intermediate_size", int),
            vocab_size=take(d, "vocab_size", int),
            # the reference's defaults for absent keys (fastgguf.c:4228, 4224)
            rms_norm_eps=take(d, "rms_norm_eps", float, 1e-6),
            rope_theta=take(theta_src, "rope_theta", float, 10000.0),
            rope_scaling=RopeScaling.from_dict(scaling_src),
            max_position_embeddings=take(d, "max_position_embeddings", int),
            tie_word_embeddings=take(d, "tie_word_embeddings", bool, False),
            torch_dtype=take(d, "torch_dtype", str, take(d, "dtype", str, "bfloat16")),
            bos_token_id=take(d, "bos_token_id", int, None),
            eos_token_ids=eos_ids,
            hidden_act=take(d, "hidden_act", str, "silu"),
        )
        cfg.validate()
        return cfg

    def to_dict(self) -> dict:
        d = {
            "architectures": [self.architecture_names[0]],
            "model_type": "llama",
            "hidden_size": self.hidden_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "intermediate_size": self.intermediate_size,
            "vocab_size": self.vocab_size,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "rope_scaling": self.rope_scaling.to_dict(),
            "max_position_embeddings": self.max_position_embeddings,
            "tie_word_embeddings": self.tie_word_embeddings,
            "torch_dtype": self.torch_dtype,
            "hidden_act": self.hidden_act,
            "attention_bias": False,
            "mlp_bias": False,
        }
        if self.bos_token_id is not None:
            d["bos_token_id"] = self.bos_token_id
        if self.eos_token_ids:
            d["eos_token_id"] = self.eos_token_ids[0] if len(self.eos_token_ids) == 1 else list(self.eos_token_ids)
        return d

    # ------------------------------------------------------------------ checking
    def validate(self) -> None:
        def positive(name):
            v = getattr(self, name)
            if v <= 0:
                raise ConfigError(f"config.json: {name} must be positive, got {v}")

        for name in ("hidden_size", "num_hidden_layers", "num_attention_heads", "num_key_value_heads",
                     "head_dim", "intermediate_size", "vocab_size", "max_position_embeddings"):
            positive(name)
        if self.num_attention_heads % self.num_key_value_heads != 0:
            raise ConfigError(
                f"config.json: num_attention_heads ({self.num_attention_heads}) must be a multiple of "
                f"num_key_value_heads ({self.num_key_value_heads})")
        if self.head_dim % 2 != 0:
            raise ConfigError(f"config.json: head_dim must be even for rotary pairs, got {self.head_dim}")
        if not (self.rms_norm_eps > 0.0):
            raise ConfigError(f"config.json: rms_norm_eps must be positive, got {self.rms_norm_eps}")
        if not (self.rope_theta > 0.0):
            raise ConfigError(f"config.json: rope_theta must be positive, got {self.rope_theta}")
        if self.hidden_act != "silu":
            raise ConfigError(f"config.json: hidden_act '{self.hidden_act}' is not supported (known: silu)")
        rs = self.rope_scaling
        if rs.rope_type == "llama3":
            if rs.factor <= 0 or rs.original_max_position_embeddings <= 0:
                raise ConfigError("config.json: rope_scaling needs positive factor and original_max_position_embeddings")
            if rs.high_freq_factor <= rs.low_freq_factor:
                raise ConfigError("config.json: rope_scaling.high_freq_factor must exceed low_freq_factor")
        for t in self.eos_token_ids:
            if not (0 <= t < self.vocab_size):
                raise ConfigError(f"config.json: eos_token_id {t} lies outside the vocabulary [0, {self.vocab_size})")

    def describe(self) -> dict:
        d = super().describe()
        d.update(q_dim=self.q_dim, kv_dim=self.kv_dim, group_size=self.group_size,
                 parameters=self.parameter_count())
        return d
