"""Weights: the safetensors format, loading by name, the random-weights mode."""
from .loader import WeightsError, load_tensors, target_dtype
from .random_init import random_tensor, random_tensors, write_model_folder
from .safetensors_io import SafetensorsError, SafetensorsFile, open_model_files, write_safetensors

__all__ = ["SafetensorsError", "SafetensorsFile", "WeightsError", "load_tensors", "open_model_files",
           "random_tensor", "random_tensors", "target_dtype", "write_model_folder", "write_safetensors"]
