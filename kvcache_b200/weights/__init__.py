from .loader import FLOAT, INTEGER, TensorSpec, WeightError, load_tensors
from .random_init import random_tensors, write_random_model
from .safetensors_io import SafetensorsError, SafetensorsFile, write_safetensors

__all__ = ["FLOAT", "INTEGER", "TensorSpec", "WeightError", "load_tensors", "random_tensors",
           "write_random_model", "SafetensorsError", "SafetensorsFile", "write_safetensors"]
