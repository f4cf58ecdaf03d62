"""Weights: the safetensors container, loading by name, random model folders."""
from .loader import FolderSource, MemorySource, TensorSource, WeightError, load_tensors
from .random_init import random_tensors, write_random_model
from .safetensors_io import SafetensorsError, SafetensorsFile, write_safetensors

__all__ = ["FolderSource", "MemorySource", "TensorSource", "WeightError", "load_tensors", "random_tensors",
           "write_random_model", "SafetensorsError", "SafetensorsFile", "write_safetensors"]
