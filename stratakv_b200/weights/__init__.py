from .safetensors_io import SafetensorsError, SafetensorsFile, write_safetensors
from .loader import WeightError, check_and_select, load_checkpoint, read_checkpoint
from .random_init import random_tensor, random_tensors, write_random_model

__all__ = ["SafetensorsError", "SafetensorsFile", "write_safetensors", "WeightError",
           "check_and_select", "load_checkpoint", "read_checkpoint", "random_tensor",
           "random_tensors", "write_random_model"]
