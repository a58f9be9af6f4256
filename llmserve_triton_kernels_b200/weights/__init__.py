from .loader import WeightError, check_tensors, read_safetensors  # noqa: F401
from .random_init import random_tensors, write_random_model  # noqa: F401
