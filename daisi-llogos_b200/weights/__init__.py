"""Safetensors input/output, the checked loader and random initialisation."""
from .loader import (WeightsError, build_model, check_tensors, load_model, random_model, random_tensors,
                     write_random_model)
from .safetensors_io import ModelFiles, SafetensorsError, SafetensorsFile, write_safetensors

__all__ = ["WeightsError", "build_model", "check_tensors", "load_model", "random_model", "random_tensors",
           "write_random_model", "ModelFiles", "SafetensorsError", "SafetensorsFile", "write_safetensors"]
