from .loader import WeightsError, load_weights, place
from .random_init import random_tensors, random_tensors_on_device, write_model_folder

__all__ = ["WeightsError", "load_weights", "place", "random_tensors", "random_tensors_on_device",
           "write_model_folder"]
