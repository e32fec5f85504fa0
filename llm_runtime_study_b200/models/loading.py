"""From a model folder (or a configuration and a seed) to a placed model."""

from __future__ import annotations

from pathlib import Path
from typing import Any, Mapping

import torch

from ..config.registry import Architecture, architecture_for, load_config
from ..parts.base import Runtime
from ..weights.checkpoint import Checkpoint, validate_manifest
from ..weights.random_init import random_state, random_tensor
from ..weights.view import TensorView
from .model import DecoderModel


def load_model_dir(model_dir: str | Path, runtime: Runtime, *, strict_dtype: bool = True) -> tuple[DecoderModel, Any, Architecture]:
    """config.json picks the architecture; headers are validated against the
    model's schema before any payload is read (mini_llm/model/base.py:276-294).
    Then every part takes its tensors one by one from the mapped files and places
    them on the device: no host copy of the checkpoint is ever made.

    ``strict_dtype``: every floating tensor must be stored in config.json's
    ``torch_dtype`` (the reference's rule, mini_llm/checkpoint.py:290, 478-481);
    off, any floating storage type is taken and converted."""

    arch, config = load_config(model_dir)
    model = DecoderModel(arch.describe(config))
    checkpoint = Checkpoint.from_model_dir(model_dir)
    validate_manifest(checkpoint, model.tensor_schema(), architecture=arch.model_type,
                      torch_dtype=getattr(config, "torch_dtype", None) if strict_dtype else None)
    model.load(checkpoint.view(), runtime)
    return model, config, arch


def random_model(
    config_dict: Mapping[str, Any], seed: int, runtime: Runtime, *, on_device: bool = False
) -> tuple[DecoderModel, Any, dict[str, torch.Tensor] | None]:
    """A model with seeded random weights, without touching the disk.  With
    ``on_device`` the values are drawn on the GPU (fast at real sizes) and are
    not returned; otherwise they are drawn on the CPU in the checkpoint's type
    and returned too, so that a plain implementation can use the same values."""

    arch = architecture_for(config_dict)
    config = arch.config_from_dict(config_dict)
    model = DecoderModel(arch.describe(config))
    schema = model.tensor_schema()
    store = {"float32": torch.float32, "bfloat16": torch.bfloat16, "float16": torch.float16}[
        config_dict.get("torch_dtype", "float32")
    ]
    if on_device:
        required = {n: s for n, s in schema.items() if not s.optional}
        model.load(
            TensorView(
                required,
                lambda name: random_tensor(name, required[name], seed, dtype=store, device=runtime.device),
            ),
            runtime,
        )
        return model, config, None
    state = random_state(schema, seed, dtype=store, include_optional=False)
    model.load(state, runtime)
    return model, config, state
