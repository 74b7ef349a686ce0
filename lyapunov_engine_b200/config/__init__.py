from .base import ConfigError, KeyReader, read_config_json
from .llama import LlamaConfig, RopeScaling
from .sulepel import SulepelConfig

__all__ = ["ConfigError", "KeyReader", "read_config_json", "LlamaConfig", "RopeScaling", "SulepelConfig"]
