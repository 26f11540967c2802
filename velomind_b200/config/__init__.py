from .base import ConfigError, KeyReader, read_config_json
from .llama import LlamaConfig
from .registry import (Architecture, architecture_name, register_architecture, registered_architectures, resolve,
                       unregister_architecture)

__all__ = ["ConfigError", "KeyReader", "read_config_json", "LlamaConfig", "Architecture", "architecture_name",
           "register_architecture", "registered_architectures", "resolve", "unregister_architecture"]
