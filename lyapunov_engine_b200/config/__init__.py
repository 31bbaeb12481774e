from .base import ConfigError, KeyReader, read_config_json
from .llama import LlamaConfig, RopeScaling

__all__ = ["ConfigError", "KeyReader", "read_config_json", "LlamaConfig", "RopeScaling"]
