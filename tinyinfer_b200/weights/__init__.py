from .loader import LoadReport, WeightError, checkpoint_index, load_weights
from .random_init import fill_random_on_device, random_tensors, write_random_model

__all__ = ["LoadReport", "WeightError", "checkpoint_index", "load_weights",
           "fill_random_on_device", "random_tensors", "write_random_model"]
