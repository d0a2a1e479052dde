from .loader import WeightStore
from .random_init import random_tensors, write_random_model
from .safetensors_io import Checkpoint, SafetensorsFile, WeightError, write_safetensors

__all__ = ["Checkpoint", "SafetensorsFile", "WeightError", "WeightStore", "random_tensors",
           "write_random_model", "write_safetensors"]
