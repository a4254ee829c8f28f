"""Weights: safetensors by tensor name, eager name/shape checks, seeded random folders."""
from .loader import (Checkpoint, ParamSpec, TensorSource, WeightError, check_names,
                     find_safetensors_files, place)
from .random_init import random_tensor, random_tensors, write_model_dir
from .safetensors_io import SafetensorsError, SafetensorsFile, read_header, save_file

__all__ = [
    "Checkpoint", "ParamSpec", "TensorSource", "WeightError", "check_names",
    "find_safetensors_files", "place", "random_tensor", "random_tensors", "write_model_dir",
    "SafetensorsError", "SafetensorsFile", "read_header", "save_file",
]
