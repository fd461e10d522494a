"""Weights by tensor name from safetensors, and the seeded random-weights mode."""
from .safetensors_io import SafetensorsError, SafetensorsFile, TensorSource, write_safetensors
from .loader import (RandomSource, TensorSpec, WeightError, check_source, fetch, fetch_many, random_tensor,
                     stored_dtype_policy, write_model_folder)

__all__ = ["SafetensorsError", "SafetensorsFile", "TensorSource", "write_safetensors",
           "RandomSource", "TensorSpec", "WeightError", "check_source", "fetch", "fetch_many", "random_tensor",
           "stored_dtype_policy", "write_model_folder"]
