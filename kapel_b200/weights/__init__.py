"""Safetensors by tensor name, one error for every misfit, and seeded random weights."""
from .loader import WeightsError, check_names, load_tensors, open_files
from .random_init import random_tensor, random_tensors, tensor_seed, write_random_model
from .safetensors import SafetensorsError, SafetensorsFile, write_safetensors
