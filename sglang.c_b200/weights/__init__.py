from .loader import DeviceStore, TensorRef, WeightError, load_checked, required_tensors
from .random_init import write_random_model
from .safetensors_io import SafetensorsError, SafetensorsFile, write_safetensors

__all__ = ["DeviceStore", "TensorRef", "WeightError", "load_checked", "required_tensors",
           "write_random_model", "SafetensorsError", "SafetensorsFile", "write_safetensors"]
