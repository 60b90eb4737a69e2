from .loader import ParamSpec, check_names, load_checkpoint, storage_dtype
from .random_init import random_tensors, write_random_model
from .safetensors_io import SafetensorsFile, open_checkpoint, write_safetensors

__all__ = ["ParamSpec", "check_names", "load_checkpoint", "storage_dtype", "random_tensors",
           "write_random_model", "SafetensorsFile", "open_checkpoint", "write_safetensors"]
