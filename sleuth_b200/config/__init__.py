"""Typed configurations and the architecture registry."""

from .base import ConfigError, read_config_json, read_fields
from .qwen3 import Qwen3Config, qwen3_model_spec
from .registry import (Architecture, find_architecture, parse_config, register_architecture,
                       registered_architectures, unregister_architecture)

register_architecture("Qwen3ForCausalLM", Qwen3Config, qwen3_model_spec, model_types=("qwen3",))

__all__ = ["ConfigError", "read_config_json", "read_fields", "Qwen3Config", "qwen3_model_spec", "Architecture",
           "find_architecture", "parse_config", "register_architecture", "registered_architectures",
           "unregister_architecture"]
