from .loader import WeightsError, kept_dtype, load_weights, merge_specs, weight_files
from .resolve import resolve_model_dir
from .random_init import random_state, random_state_on_device, write_random_model
from .safetensors_io import SafetensorsFile, save_safetensors

__all__ = ["WeightsError", "kept_dtype", "load_weights", "merge_specs", "weight_files", "random_state", "random_state_on_device",
           "write_random_model", "SafetensorsFile", "save_safetensors", "resolve_model_dir"]
