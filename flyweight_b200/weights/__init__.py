from .loader import TensorDecl, WeightError, bind, load_checkpoint
from .random_init import random_tensor, random_tensors, write_model_dir
from .safetensors_io import (SafetensorsError, load_file, load_model_tensors, read_header,
                             save_file)

__all__ = [
    "TensorDecl", "WeightError", "bind", "load_checkpoint", "random_tensor", "random_tensors",
    "write_model_dir", "SafetensorsError", "load_file", "load_model_tensors", "read_header",
    "save_file",
]
