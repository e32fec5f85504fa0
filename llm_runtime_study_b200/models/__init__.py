from . import qwen3  # registers the architecture
from .description import LayerDescription, ModelDescription, tensor_schema
from .loading import load_model_dir, random_model
from .model import DecoderModel

__all__ = [
    "DecoderModel", "LayerDescription", "ModelDescription", "load_model_dir", "random_model", "tensor_schema",
]
