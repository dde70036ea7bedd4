"""Typed configurations and the architecture registry."""

from .base import ConfigError, read_config_json
from .qwen3 import Qwen3Config
from .registry import REGISTRY, ModelFamily, family_of, load_config, register_architecture

__all__ = ["ConfigError", "Qwen3Config", "REGISTRY", "ModelFamily", "family_of", "load_config",
           "read_config_json", "register_architecture"]
