"""Weights: safetensors files, loading by tensor name, random weights."""
from .safetensors_io import Checkpoint, SafetensorsError, SafetensorsFile, write_safetensors
from .loader import WeightError, check_checkpoint, load_weights
from .random_init import bind_random_weights, random_tensors, write_random_model

__all__ = ["Checkpoint", "SafetensorsError", "SafetensorsFile", "write_safetensors", "WeightError",
           "check_checkpoint", "load_weights", "bind_random_weights", "random_tensors",
           "write_random_model"]
