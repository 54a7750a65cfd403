"""Weights from safetensors by tensor name, and the random-weights mode."""
from .loader import DictSource, WeightError, WeightSource, check_against, stored_precision
from .random_init import write_random_model
from .safetensors_io import Checkpoint, SafetensorsError, SafetensorsFile, save_tensors, write_safetensors

__all__ = ["Checkpoint", "DictSource", "SafetensorsError", "SafetensorsFile", "WeightError", "WeightSource", "check_against",
           "save_tensors", "stored_precision", "write_random_model", "write_safetensors"]
