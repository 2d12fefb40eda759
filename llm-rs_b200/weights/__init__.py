"""Weights: the safetensors container, loading by name with full error reports, random weights."""
from .safetensors_io import SafetensorsFile, WeightFileError, open_model_files, save_file
from .loader import WeightError, load_weights
from .random_init import random_tensors, write_random_model

__all__ = ["SafetensorsFile", "WeightFileError", "open_model_files", "save_file", "WeightError", "load_weights",
           "random_tensors", "write_random_model"]
