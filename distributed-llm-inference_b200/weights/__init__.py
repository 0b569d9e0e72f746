from .loader import CheckpointError, TensorDecl, load_tensors
from .random_init import random_tensors, write_model_dir
from .safetensors_io import SafetensorsFile, write_safetensors

__all__ = ["CheckpointError", "SafetensorsFile", "TensorDecl", "load_tensors", "random_tensors", "write_model_dir", "write_safetensors"]
