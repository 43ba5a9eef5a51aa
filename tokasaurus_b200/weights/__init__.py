from tokasaurus_b200.weights.loader import WeightLoadError, load_weights, target_dtype  # noqa: F401
from tokasaurus_b200.weights.random_init import random_tensors, write_model_folder  # noqa: F401
