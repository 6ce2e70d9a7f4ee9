from .base import ConfigError, ModelConfig, read_config_json
from .qwen3 import Qwen3Config

__all__ = ["ConfigError", "ModelConfig", "Qwen3Config", "read_config_json"]
