"""Weights: safetensors files, named tensor sources, the binding check, random models."""
from .loader import RandomSource, SafetensorsSource, TensorNeed, TensorSource, bind_check
from .random_init import write_random_model
from .safetensors import SafetensorsFile, write_safetensors

__all__ = ["RandomSource", "SafetensorsSource", "TensorNeed", "TensorSource", "bind_check", "write_random_model",
           "SafetensorsFile", "write_safetensors"]
