from .loader import WeightError, check_checkpoint, load_checkpoint  # noqa: F401
from .random_init import random_tensor, random_weights, write_random_model  # noqa: F401
from .safetensors_io import ModelFiles, SafetensorsFile, WeightFileError, write_safetensors  # noqa: F401
