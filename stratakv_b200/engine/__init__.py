from .engine import Engine, StepEntry, StepError
from .model import Model, cache_requests, expected_tensors

__all__ = ["Engine", "StepEntry", "StepError", "Model", "cache_requests", "expected_tensors"]
