"""A B200-native inference engine for Qwen3 dense: typed configuration and
architecture registry, safetensors weights, a model assembled from parts, a
paged cache manager, one step function for mixed batches, a scheduler, sampling,
and hand-written CUDA kernels for sm_100a."""

from . import models as _models  # noqa: F401  (registers the built-in architecture)
from .errors import (
    CheckpointError, CheckpointValidationError, ConfigError, EngineError, GenerationError,
    KernelError, KVCacheError, RegistryError, SamplingError,
)

__version__ = "0.1.0"

__all__ = [
    "CheckpointError", "CheckpointValidationError", "ConfigError", "EngineError", "GenerationError",
    "KernelError", "KVCacheError", "RegistryError", "SamplingError", "__version__",
]
