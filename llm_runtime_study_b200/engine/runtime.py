"""Resolution of device and dtype, and assembly of model + cache + step runner."""

from __future__ import annotations

from dataclasses import dataclass
from pathlib import Path
from typing import Any, Mapping

import torch

from ..cache.manager import CacheManager
from ..errors import EngineError
from ..models.loading import load_model_dir, random_model
from ..models.model import DecoderModel
from ..parts.base import Runtime
from .step import StepRunner

_DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def resolve_device(requested: str | torch.device = "auto") -> torch.device:
    """Only CUDA devices run this engine (the reference also accepts cpu and mps,
    mini_llm/engine.py:70-103; those backends are not built here)."""

    if requested == "auto":
        requested = "cuda"
    try:
        device = torch.device(requested)
    except (TypeError, RuntimeError) as exc:
        raise EngineError(f"invalid device {requested!r}") from exc
    if device.type != "cuda":
        raise EngineError(f"unsupported device {device}; this engine runs on CUDA devices only")
    if not torch.cuda.is_available():
        raise EngineError("CUDA was requested but is unavailable; this engine has no CPU path")
    if device.index is not None and device.index >= torch.cuda.device_count():
        raise EngineError(
            f"CUDA device index {device.index} is unavailable; found {torch.cuda.device_count()} CUDA device(s)"
        )
    if device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    return device


def resolve_dtype(requested: str | torch.dtype = "auto") -> torch.dtype:
    """``auto`` is bfloat16, the serving type (the reference resolves ``auto`` to
    float16 on accelerators, mini_llm/engine.py:106-132; float16 is not built here)."""

    if requested == "auto":
        return torch.bfloat16
    if isinstance(requested, torch.dtype):
        dtype = requested
    elif isinstance(requested, str) and requested in _DTYPES:
        dtype = _DTYPES[requested]
    else:
        raise EngineError(f"unsupported dtype {requested!r}; expected auto, bfloat16 or float32")
    if dtype not in _DTYPES.values():
        raise EngineError(f"unsupported dtype {dtype}; expected bfloat16 or float32")
    return dtype


@dataclass
class LoadedModel:
    model: DecoderModel
    config: Any
    runtime: Runtime
    weights: Mapping[str, torch.Tensor] | None = None  # CPU copies, random mode only

    def make_runner(
        self, *, max_tokens: int, page_size: int, max_requests: int, max_seq_len: int | None = None,
        max_step_tokens: int | None = None,
    ) -> StepRunner:
        """``max_step_tokens``: the most tokens one step will ever carry, if the caller knows it (a scheduler's
        token budget); groups of layers that read a window only are then given pools for the window."""

        description = self.model.description
        manager = CacheManager(
            self.model.cache_layout(), max_tokens=max_tokens, page_size=page_size,
            max_requests=max_requests, dtype=self.runtime.dtype, device=self.runtime.device,
            max_seq_len=max_seq_len or description.max_positions, max_step_tokens=max_step_tokens,
        )
        return StepRunner(
            self.model, manager, self.runtime, vocab_size=description.vocab_size,
            max_positions=description.max_positions,
        )


def load(model_dir: str | Path, *, device="auto", dtype="auto", strict_dtype: bool = True) -> LoadedModel:
    from ..config.registry import load_config

    load_config(model_dir)  # a bad folder or config.json is reported before anything about the device
    runtime = Runtime(resolve_device(device), resolve_dtype(dtype))
    with torch.cuda.device(runtime.device):
        model, config, _ = load_model_dir(model_dir, runtime, strict_dtype=strict_dtype)
    return LoadedModel(model, config, runtime)


def load_random(config_dict: Mapping[str, Any], seed: int, *, device="auto", dtype="auto", on_device=False) -> LoadedModel:
    runtime = Runtime(resolve_device(device), resolve_dtype(dtype))
    with torch.cuda.device(runtime.device):
        model, config, weights = random_model(config_dict, seed, runtime, on_device=on_device)
    return LoadedModel(model, config, runtime, weights)
