"""Weights by tensor name: safetensors container, checks, random generation."""
from .loader import (TensorDecl, WeightsError, check_tensors, load_tensors, random_tensors, write_model_folder)
from .safetensors_io import SafetensorsError, SafetensorsFile, write_safetensors

__all__ = ["TensorDecl", "WeightsError", "check_tensors", "load_tensors", "random_tensors", "write_model_folder",
           "SafetensorsError", "SafetensorsFile", "write_safetensors"]
