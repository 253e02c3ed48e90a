"""Weights: safetensors by tensor name, and a seeded random-weights mode."""
from .loader import WeightError, list_tensors, load_weights
from .random_init import bind_random, random_tensors, write_random_model

__all__ = ["WeightError", "list_tensors", "load_weights", "bind_random", "random_tensors", "write_random_model"]
