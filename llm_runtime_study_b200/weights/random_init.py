"""Seeded random weights, in memory or written out as a model folder.

The reference has no such mode (its tests build a module under
``torch.manual_seed``, tests/test_cache.py:78-79).  Here every tensor of the
schema is filled from its own generator, seeded by ``(seed, tensor name)``, so
the values do not depend on the order of generation or on which other tensors
exist; they are drawn in float32 and rounded once to the storage type.
"""

from __future__ import annotations

import hashlib
import json
from pathlib import Path
from typing import Any, Mapping

import torch

from .checkpoint import TensorSpec
from .safetensors_io import write_file

_TORCH_DTYPES = {
    "float32": torch.float32,
    "bfloat16": torch.bfloat16,
    "float16": torch.float16,
}


def _tensor_seed(seed: int, name: str) -> int:
    digest = hashlib.sha256(f"{seed}:{name}".encode("utf-8")).digest()
    return int.from_bytes(digest[:8], "little") & 0x7FFF_FFFF_FFFF_FFFF


def random_tensor(
    name: str, spec: TensorSpec, seed: int, *, dtype: torch.dtype, device: str | torch.device = "cpu"
) -> torch.Tensor:
    """One tensor of the schema.  CPU and CUDA generators give different
    streams; each is reproducible on its own device."""

    device = torch.device(device)
    if spec.kind == "int":
        return torch.zeros(spec.shape, dtype=torch.int32, device=device)
    generator = torch.Generator(device=device)
    generator.manual_seed(_tensor_seed(seed, name))
    if spec.init == "zeros":
        values = torch.zeros(spec.shape, dtype=torch.float32, device=device)
    else:
        values = torch.empty(spec.shape, dtype=torch.float32, device=device)
        values.normal_(0.0, spec.std, generator=generator)
        if spec.init == "one_plus_normal":
            values += 1.0
        elif spec.init != "normal":
            raise ValueError(f"unknown init {spec.init!r} for {name}")
    return values.to(dtype)


def random_state(
    specs: Mapping[str, TensorSpec], seed: int, *, dtype: torch.dtype,
    device: str | torch.device = "cpu", include_optional: bool = True,
) -> dict[str, torch.Tensor]:
    return {
        name: random_tensor(name, spec, seed, dtype=dtype, device=device)
        for name, spec in sorted(specs.items())
        if include_optional or not spec.optional
    }


def write_random_model(
    model_dir: str | Path, config_dict: Mapping[str, Any], seed: int, *, shards: int = 1
) -> Path:
    """Write ``config.json`` and ``model.safetensors`` (or ``shards`` files and
    an index) for the architecture that ``config_dict`` names.  Optional tensors
    (a tied head) are left out, so the folder exercises the tied path."""

    from ..config import architecture_for
    from ..models.description import tensor_schema

    arch = architecture_for(config_dict)
    config = arch.config_from_dict(config_dict)
    specs = tensor_schema(arch.describe(config))
    dtype = _TORCH_DTYPES[config_dict.get("torch_dtype", "float32")]
    state = random_state(specs, seed, dtype=dtype, include_optional=False)

    model_path = Path(model_dir)
    model_path.mkdir(parents=True, exist_ok=True)
    (model_path / "config.json").write_text(json.dumps(dict(config_dict), indent=2), encoding="utf-8")
    names = sorted(state)
    if shards <= 1:
        write_file(model_path / "model.safetensors", state)
    else:
        weight_map: dict[str, str] = {}
        per = (len(names) + shards - 1) // shards
        for s in range(shards):
            part = names[s * per : (s + 1) * per]
            if not part:
                continue
            file_name = f"model-{s + 1:05d}-of-{shards:05d}.safetensors"
            write_file(model_path / file_name, {n: state[n] for n in part})
            weight_map.update({n: file_name for n in part})
        (model_path / "model.safetensors.index.json").write_text(
            json.dumps({"metadata": {}, "weight_map": weight_map}, indent=2), encoding="utf-8"
        )
    return model_path
