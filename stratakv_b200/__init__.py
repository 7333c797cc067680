"""A small single-GPU generation library for the dense Llama decoder on B200 (sm_100a)."""
from . import models as _models  # noqa: F401
from .config import ConfigError, EngineConfig, LlamaConfig, load_config
from .engine import Engine, StepEntry, StepError

__all__ = ["ConfigError", "EngineConfig", "LlamaConfig", "load_config", "Engine", "StepEntry", "StepError"]
__version__ = "0.1.0"
