"""Weights: the safetensors container, binding by tensor name, and seeded random models."""
from .loader import LazyTensors, WeightDecl, WeightError, load_checkpoint, open_checkpoint
from .random_init import random_tensor, random_tensors, write_model_folder
from .safetensors_io import SafetensorsError, SafetensorsFile, shard_paths, write_safetensors

__all__ = ["LazyTensors", "WeightDecl", "WeightError", "load_checkpoint", "open_checkpoint", "random_tensor", "random_tensors", "write_model_folder",
           "SafetensorsError", "SafetensorsFile", "shard_paths", "write_safetensors"]
