from .safetensors_io import Checkpoint, SafetensorsError, SafetensorsFile, TensorDict, write_safetensors
from .loader import WeightBinder, WeightError, expected_tensors, memory_dtype
from .random_init import random_tensors, write_random_model

__all__ = ["Checkpoint", "SafetensorsError", "SafetensorsFile", "TensorDict", "write_safetensors", "WeightBinder",
           "WeightError", "expected_tensors", "memory_dtype", "random_tensors", "write_random_model"]
