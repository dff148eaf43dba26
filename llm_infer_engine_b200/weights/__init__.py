from .loader import WeightsError, build_model, compare, load_weights, target_dtype
from .random_init import random_tensors, scratch_folder, write_random_model
from .safetensors_io import SafetensorsError, SafetensorsFile, open_model_files, save_file

__all__ = ["WeightsError", "build_model", "compare", "load_weights", "target_dtype", "random_tensors",
           "write_random_model", "scratch_folder", "SafetensorsError", "SafetensorsFile", "open_model_files", "save_file"]
