from .checkpoint import Checkpoint, TensorSpec, validate_manifest
from .random_init import random_state, random_tensor, write_random_model
from .safetensors_io import TensorInfo, map_tensor, read_header, read_tensors, write_file

__all__ = [
    "Checkpoint", "TensorInfo", "TensorSpec", "random_state", "random_tensor",
    "map_tensor", "read_header", "read_tensors", "validate_manifest", "write_file", "write_random_model",
]
