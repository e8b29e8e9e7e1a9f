"""Weights: safetensors by tensor name, one clear error, a random-weights mode."""

from .loader import WeightError, check_state, load_tensors, plan_loading
from .random_init import RandomOptions, random_state, random_tensor, write_model_folder
from .safetensors_io import Checkpoint, SafetensorsFile, write_safetensors
from .spec import Cat, Init, Name, Stack, TensorSpec, device_dtype

__all__ = [
    "WeightError", "check_state", "load_tensors", "plan_loading",
    "RandomOptions", "random_state", "random_tensor", "write_model_folder",
    "Checkpoint", "SafetensorsFile", "write_safetensors",
    "Cat", "Init", "Name", "Stack", "TensorSpec", "device_dtype",
]
