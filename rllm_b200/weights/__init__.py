from .loader import WeightError, expected_tensors, load_weights
from .random_init import init_random_weights, random_tensors, write_random_model
from .safetensors_io import TensorStore, WeightFileError, write_safetensors

__all__ = ["WeightError", "expected_tensors", "load_weights", "init_random_weights",
           "random_tensors", "write_random_model", "TensorStore", "WeightFileError",
           "write_safetensors"]
