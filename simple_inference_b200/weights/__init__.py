from .loader import WeightError, load_tensors
from .random_init import model_for_config, random_tensors, write_random_model

__all__ = ["WeightError", "load_tensors", "model_for_config", "random_tensors",
           "write_random_model"]
