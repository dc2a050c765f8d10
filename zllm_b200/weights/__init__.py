from .safetensors_io import SafetensorsFile, open_model_files, write_safetensors
from .loader import check_names, load_checked, target_dtype
from .random_init import random_state, random_tensor, write_random_model

__all__ = ["SafetensorsFile", "open_model_files", "write_safetensors", "check_names", "load_checked",
           "target_dtype", "random_state", "random_tensor", "write_random_model"]
