"""Typed configurations, one class per architecture, chosen by ``architectures[0]``."""
from .base import ConfigError, ModelConfig, architecture_name, read_config_json
from .llama import LlamaConfig, RopeScaling

__all__ = ["ConfigError", "ModelConfig", "LlamaConfig", "RopeScaling", "architecture_name", "read_config_json"]
