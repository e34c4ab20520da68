from .loader import WeightError, check_tensors, read_checkpoint
from .random_init import random_tensors, write_model_dir

__all__ = ["WeightError", "check_tensors", "random_tensors", "read_checkpoint", "write_model_dir"]
