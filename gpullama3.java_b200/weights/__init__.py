"""Weights: the safetensors container, binding by tensor name, and the random-weights mode."""
from .safetensors_io import SafetensorsFile, WeightError, open_model_files, write_safetensors
from .loader import ParamSpec, check_names_and_shapes, load_checkpoint_tensors, storage_dtype
from .random_init import random_checkpoint, random_tensor, write_random_model

__all__ = ["SafetensorsFile", "WeightError", "open_model_files", "write_safetensors", "ParamSpec",
           "check_names_and_shapes", "load_checkpoint_tensors", "storage_dtype", "random_checkpoint",
           "random_tensor", "write_random_model"]
