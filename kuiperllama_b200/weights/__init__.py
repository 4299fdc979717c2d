"""Weights: safetensors by tensor name, and random model folders."""
from .loader import TensorDecl, WeightsError, load_tensors, stored_dtype
from .safetensors_io import SafetensorsFile, SafetensorsFormatError, write_safetensors

__all__ = ["TensorDecl", "WeightsError", "load_tensors", "stored_dtype", "SafetensorsFile",
           "SafetensorsFormatError", "write_safetensors"]
