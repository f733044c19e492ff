from .loader import ParamSpec, WeightsError, check_names, load_weights, target_dtype
from .random_init import random_state_dict, random_tensor, write_random_model
from .safetensors_io import SafetensorsError, SafetensorsFile, open_model_files, save_file

__all__ = ["ParamSpec", "WeightsError", "check_names", "load_weights", "target_dtype",
           "random_state_dict", "random_tensor", "write_random_model", "SafetensorsError",
           "SafetensorsFile", "open_model_files", "save_file"]
