from .loader import WeightMismatchError, load_checked
from .random_init import write_random_model
from .safetensors_io import SafetensorsFile, save_tensors

__all__ = ["WeightMismatchError", "load_checked", "write_random_model", "SafetensorsFile",
           "save_tensors"]
