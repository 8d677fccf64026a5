from .loader import WeightError, WeightSpec, check_tensors, load_weights
from .random_init import draw_tensor, draw_tensors, write_random_model
from .safetensors_io import (SafetensorsError, SafetensorsFile, open_model_shards,
                             write_safetensors)

__all__ = [
    "WeightError", "WeightSpec", "check_tensors", "load_weights", "draw_tensor", "draw_tensors",
    "write_random_model", "SafetensorsError", "SafetensorsFile", "open_model_shards",
    "write_safetensors",
]
