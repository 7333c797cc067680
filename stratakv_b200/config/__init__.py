from .llama import ConfigError, LlamaConfig
from .registry import (Architecture, known_architectures, load_config, read_config_json,
                       register_architecture, resolve_architecture)
from .engine import EngineConfig

__all__ = ["ConfigError", "LlamaConfig", "EngineConfig", "Architecture", "known_architectures",
           "load_config", "read_config_json", "register_architecture", "resolve_architecture"]
