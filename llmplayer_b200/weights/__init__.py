"""Weights: the safetensors container, loading by name, seeded random models."""
from .loader import load_tensors
from .random_init import random_tensors, write_random_model
from .safetensors_io import SafetensorsFile, write_safetensors

__all__ = ["SafetensorsFile", "load_tensors", "random_tensors", "write_random_model", "write_safetensors"]
