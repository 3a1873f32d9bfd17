from .loader import TensorSpec, WeightsError, checkpoint_files, load_weights
from .random_init import random_tensor, random_weights, write_model_folder
from .safetensors_io import SafetensorsError, SafetensorsFile, write_safetensors

__all__ = [
    "SafetensorsError",
    "SafetensorsFile",
    "TensorSpec",
    "WeightsError",
    "checkpoint_files",
    "load_weights",
    "random_tensor",
    "random_weights",
    "write_model_folder",
    "write_safetensors",
]
