"""Weights: reading safetensors by name, and seeded random models."""

from .loader import load_tensors
from .needs import TensorNeed, WeightError
from .random_init import random_tensor, random_tensors, write_random_model

__all__ = ["TensorNeed", "WeightError", "load_tensors", "random_tensor", "random_tensors", "write_random_model"]
