from .loader import Expected, WeightsError, check_names, kept_dtype, load_from_folder, load_from_tensors
from .random_init import random_tensors, write_model_folder
from .safetensors_io import SafetensorsError, SafetensorsFile, open_model_shards, write_safetensors

__all__ = ["Expected", "WeightsError", "check_names", "kept_dtype", "load_from_folder", "load_from_tensors",
           "random_tensors", "write_model_folder", "SafetensorsError", "SafetensorsFile", "open_model_shards",
           "write_safetensors"]
