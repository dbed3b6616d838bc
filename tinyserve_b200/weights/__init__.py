from .loader import WeightError, check_checkpoint, expected_tensors, load_weights
from .random_init import fill_random_on_device, write_random_model

__all__ = ["WeightError", "check_checkpoint", "expected_tensors", "load_weights",
           "fill_random_on_device", "write_random_model"]
