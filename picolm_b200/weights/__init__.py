from .loader import WeightsError, check_checkpoint, load_weights
from .random_init import random_tensors, write_random_model
from .safetensors_io import Checkpoint, SafetensorsError, SafetensorsFile, save_safetensors

__all__ = ["WeightsError", "check_checkpoint", "load_weights", "random_tensors", "write_random_model",
           "Checkpoint", "SafetensorsError", "SafetensorsFile", "save_safetensors"]
