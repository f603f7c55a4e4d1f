"""Safetensors IO, checked loading by tensor name, and random-weights mode."""
from .loader import TensorSpec, WeightError, WeightSource, check_tensors, load_weights, stored_dtype
from .random_init import random_tensors, write_random_model
from .safetensors_io import SafetensorsError, SafetensorsFile, open_model_shards, write_safetensors

__all__ = ["TensorSpec", "WeightError", "WeightSource", "check_tensors", "load_weights", "stored_dtype", "random_tensors",
           "write_random_model", "SafetensorsError", "SafetensorsFile", "open_model_shards",
           "write_safetensors"]
