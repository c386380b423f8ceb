"""Weights: the safetensors container, loading by name, seeded random models."""
from .loader import SafetensorsFolder, WeightDecl, WeightError, kept_dtype, load_weights
from .random_init import RandomSource, random_tensor, write_random_model
from .safetensors_io import SafetensorsError, SafetensorsFile, write_safetensors

__all__ = ["SafetensorsFolder", "WeightDecl", "WeightError", "kept_dtype", "load_weights",
           "RandomSource", "random_tensor", "write_random_model", "SafetensorsError",
           "SafetensorsFile", "write_safetensors"]
