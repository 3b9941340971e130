"""Safetensors by tensor name, one error for every misfit, and seeded random weights."""
from .loader import WeightSource, WeightsError, check_names, load_tensors, open_files, open_weights
from .random_init import RandomSource, random_tensor, random_tensors, tensor_seed, write_random_model
from .safetensors import SafetensorsError, SafetensorsFile, write_safetensors
