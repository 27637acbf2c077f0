from .safetensors_io import TensorFiles, TensorInfo, WeightFormatError, index_file, write_file
from .loader import Checkpoint, TensorNeed, WeightError, check_tensors, kept_dtype
from .random_init import random_tensors, write_random_model

__all__ = ["TensorFiles", "TensorInfo", "WeightFormatError", "index_file", "write_file",
           "Checkpoint", "TensorNeed", "WeightError", "check_tensors", "kept_dtype",
           "random_tensors", "write_random_model"]
