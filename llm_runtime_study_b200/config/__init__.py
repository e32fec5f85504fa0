from .fields import read_config_dict, required, optional
from .qwen3 import Qwen3Config
from .registry import (
    Architecture,
    architecture_for,
    load_config,
    register_architecture,
    registered_architectures,
)

__all__ = [
    "Architecture",
    "Qwen3Config",
    "architecture_for",
    "load_config",
    "optional",
    "read_config_dict",
    "register_architecture",
    "registered_architectures",
    "required",
]
