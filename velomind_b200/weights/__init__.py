from .loader import WeightError, WeightSpec, check_and_bind, load_weights
from .safetensors_io import SafetensorsError, load_file, read_header, save_file
from .synthetic import random_tensors, write_random_model

__all__ = ["WeightError", "WeightSpec", "check_and_bind", "load_weights", "SafetensorsError", "load_file",
           "read_header", "save_file", "random_tensors", "write_random_model"]
