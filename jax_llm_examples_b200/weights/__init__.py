from .loader import TensorSpec, WeightError, check_tensors, load_tensors
from .random_init import random_tensor, random_tensors, write_random_model

__all__ = ["TensorSpec", "WeightError", "check_tensors", "load_tensors", "random_tensor", "random_tensors",
           "write_random_model"]
