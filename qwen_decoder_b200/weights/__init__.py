from .loader import TensorSource, TensorSpec, WeightError, check_tensors, load_into, storage_dtype
from .random_init import random_tensor, random_tensors, write_random_model
from .safetensors_io import SafetensorsError, SafetensorsFile, open_model_tensors, save_safetensors

__all__ = [
    "TensorSource", "TensorSpec", "WeightError", "check_tensors", "load_into", "storage_dtype",
    "random_tensor", "random_tensors", "write_random_model", "SafetensorsError", "SafetensorsFile",
    "open_model_tensors", "save_safetensors",
]
