from .loader import WeightError, check_and_place, checkpoint_files, load_weights, read_checkpoint
from .random_init import random_tensors, write_random_model

__all__ = ["WeightError", "check_and_place", "checkpoint_files", "load_weights", "read_checkpoint",
           "random_tensors", "write_random_model"]
