"""Weights: safetensors by tensor name, and the random-weights mode."""
from .spec import EMBEDDING, INT_TABLE, MATRIX, NORM, TensorSpec
from .safetensors_io import Checkpoint, SafetensorsError, write_safetensors
from .loader import WeightError, load_tensors, resident_dtype
from .random_init import random_tensor, random_tensors, write_random_model

__all__ = ["EMBEDDING", "INT_TABLE", "MATRIX", "NORM", "TensorSpec", "Checkpoint",
           "SafetensorsError", "write_safetensors", "WeightError", "load_tensors",
           "resident_dtype", "random_tensor", "random_tensors", "write_random_model"]
