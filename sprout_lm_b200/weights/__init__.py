from .checkpoint import Checkpoint, WeightError
from .random_init import random_tensor, write_random_model
from .safetensors_io import SafetensorsError, SafetensorsFile, write_safetensors

__all__ = ["Checkpoint", "WeightError", "SafetensorsError", "SafetensorsFile", "write_safetensors",
           "write_random_model", "random_tensor"]
