from .loader import TensorSpec, WeightError, check_tensors, load_tensors
from .random_init import random_tensors, write_random_model
from .safetensors_io import SafetensorsError, SafetensorsFile, write_safetensors

__all__ = ["TensorSpec", "WeightError", "SafetensorsError", "SafetensorsFile", "check_tensors", "load_tensors",
           "random_tensors", "write_random_model", "write_safetensors"]
