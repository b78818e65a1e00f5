"""Reading weights by tensor name, and writing seeded random model folders."""

from .loader import WeightError, check, load_into
from .random_init import random_tensors, write_random_model
from .safetensors import Checkpoint, SafetensorsError, SafetensorsFile, read_safetensors, write_safetensors

__all__ = ["WeightError", "check", "load_into", "random_tensors", "write_random_model", "Checkpoint",
           "SafetensorsError", "SafetensorsFile", "read_safetensors", "write_safetensors"]
