"""Typed errors, one per layer of the engine.

The reference raises one error class per layer and its command line maps all of
them to exit code 2 (mini_llm/cli.py:273-284).  The same classes exist here so a
caller can tell a bad ``config.json`` from a bad checkpoint from a full cache.
"""

from __future__ import annotations


class ConfigError(ValueError):
    """``config.json`` is missing, malformed, or names an unsupported option."""


class CheckpointError(ValueError):
    """A checkpoint file, shard or index cannot be read."""


class CheckpointValidationError(CheckpointError):
    """Tensor names, shapes or dtypes do not match the configuration."""


class KVCacheError(RuntimeError):
    """The cache manager cannot satisfy a request (pool exhausted, bad handle)."""


class GenerationError(ValueError):
    """A request cannot be scheduled (too long, empty, bad limits)."""


class SamplingError(ValueError):
    """Sampling options or logits are invalid."""


class EngineError(ValueError):
    """Device, dtype or context length is unsupported."""


class KernelError(RuntimeError):
    """A CUDA kernel refused its sizes, or the native library is unavailable."""


class RegistryError(KeyError):
    """A part kind or an architecture name is not registered."""
