from .safetensors_io import SafetensorsFile, write_safetensors
from .state_map import StateMap, TensorNeed
from .random_init import random_state, random_tensor, write_model_folder

__all__ = ["SafetensorsFile", "write_safetensors", "StateMap", "TensorNeed", "random_state",
           "random_tensor", "write_model_folder"]
