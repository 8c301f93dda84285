"""Weights: safetensors container, by-name binding, random-weights mode."""
from .loader import bind_tensors, load_model_tensors, model_param_decls, place_tensor
from .random_init import random_tensors, write_random_model
from .safetensors_io import read_model_tensors, read_safetensors_file, write_safetensors_file

__all__ = ["bind_tensors", "load_model_tensors", "model_param_decls", "place_tensor",
           "random_tensors", "write_random_model", "read_model_tensors",
           "read_safetensors_file", "write_safetensors_file"]
