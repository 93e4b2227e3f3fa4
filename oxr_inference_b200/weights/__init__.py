from oxr_inference_b200.weights.loader import WeightError, checkpoint_files, load_weights
from oxr_inference_b200.weights.random_init import fill_random, random_tensor, shape_only_model, write_random_model

__all__ = ["WeightError", "checkpoint_files", "fill_random", "load_weights", "random_tensor", "shape_only_model",
           "write_random_model"]
