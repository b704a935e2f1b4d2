from .safetensors_io import ModelFolder, SafetensorsFile, WeightsError, write_safetensors
from .loader import fill_from_folder, load_model, torch_dtype
from .random_init import fill_random_, write_random_model

__all__ = ["ModelFolder", "SafetensorsFile", "WeightsError", "write_safetensors", "fill_from_folder",
           "load_model", "torch_dtype", "fill_random_", "write_random_model"]
