from .loader import WeightStore
from .random_init import DeviceRandomStore, counter_normal, open_weight_store, random_tensors, write_random_model
from .safetensors_io import Checkpoint, SafetensorsFile, WeightError, write_safetensors

__all__ = ["Checkpoint", "DeviceRandomStore", "SafetensorsFile", "WeightError", "WeightStore", "counter_normal",
           "open_weight_store", "random_tensors", "write_random_model", "write_safetensors"]
