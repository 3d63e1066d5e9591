from .safetensors_io import SafetensorsFile, save_safetensors, SafetensorsError
from .loader import load_weights, WeightError
from .random_init import write_random_model, random_weights, random_tensor

__all__ = ["SafetensorsFile", "save_safetensors", "SafetensorsError", "load_weights", "WeightError",
           "write_random_model", "random_weights", "random_tensor"]
