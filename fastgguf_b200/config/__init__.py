"""Typed configurations, chosen by ``architectures[0]`` of config.json (read and checked by the C++ host)."""
from .base import ConfigError, ModelConfig, architecture_name, read_config_json
from .llama import LlamaConfig

__all__ = ["ConfigError", "ModelConfig", "LlamaConfig", "architecture_name", "read_config_json"]
