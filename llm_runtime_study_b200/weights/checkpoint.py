"""Checkpoint manifest and its validation against a tensor schema.

Locating rules follow mini_llm/checkpoint.py:83-137 (``model.safetensors`` if
present, else ``model.safetensors.index.json`` whose ``weight_map`` names the
shards).  Validation follows mini_llm/checkpoint.py:453-487: every name, shape and
storage type is checked before any payload is read, and *all* problems are reported
in one error.  The schema itself is not written here: each part of the model declares
the tensors it owns (``Part.tensor_specs``), and the model description joins them.
"""

from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Iterable, Mapping

import torch

from ..errors import CheckpointError, CheckpointValidationError
from .safetensors_io import FLOAT_DTYPES, INT_DTYPES, TensorInfo, map_tensor, read_header, read_tensors
from .view import TensorView

# config.json's torch_dtype -> the safetensors type every floating tensor must then be stored in
STORAGE_NAME = {"float32": "F32", "bfloat16": "BF16", "float16": "F16"}


@dataclass(frozen=True, slots=True)
class TensorSpec:
    """What the model expects of one stored tensor.

    ``kind`` is ``"float"`` (converted to the run type at placement) or ``"int"``
    (index tables; placed as int32).  ``init`` tells
    the random-weights mode how to fill it: ``"normal"`` N(0, std),
    ``"one_plus_normal"`` 1 + N(0, std), ``"zeros"``.  ``optional`` tensors may
    be absent (a tied output head).
    """

    shape: tuple[int, ...]
    kind: str = "float"
    init: str = "normal"
    std: float = 0.02
    optional: bool = False


class Checkpoint:
    """Merged, name-sorted manifest of a single-file or sharded checkpoint."""

    def __init__(self, infos: Iterable[TensorInfo], source: Path) -> None:
        self.source = source
        self.manifest: tuple[TensorInfo, ...] = tuple(sorted(infos, key=lambda i: i.name))
        self._by_name = {info.name: info for info in self.manifest}

    @classmethod
    def from_model_dir(cls, model_dir: str | Path) -> "Checkpoint":
        model_path = Path(model_dir)
        single = model_path / "model.safetensors"
        if single.is_file():
            return cls(read_header(single), single)
        index = model_path / "model.safetensors.index.json"
        if index.is_file():
            return cls._from_index(index)
        raise CheckpointError(
            "model directory contains neither model.safetensors nor "
            f"model.safetensors.index.json: {model_path}"
        )

    @classmethod
    def _from_index(cls, index_path: Path) -> "Checkpoint":
        try:
            index = json.loads(index_path.read_text(encoding="utf-8"))
        except json.JSONDecodeError as exc:
            raise CheckpointError(f"invalid JSON in {index_path}: {exc}") from exc
        weight_map = index.get("weight_map") if isinstance(index, dict) else None
        if not isinstance(weight_map, dict) or not weight_map or not all(
            isinstance(k, str) and isinstance(v, str) for k, v in weight_map.items()
        ):
            raise CheckpointError(f"weight_map must be a non-empty object of strings: {index_path}")
        shards: dict[str, dict[str, TensorInfo]] = {}
        for shard in dict.fromkeys(weight_map.values()):
            shard_path = index_path.parent / shard
            if not shard_path.is_file():
                raise CheckpointError(f"checkpoint shard does not exist: {shard_path}")
            shards[shard] = {info.name: info for info in read_header(shard_path)}
        infos = []
        for name, shard in weight_map.items():
            info = shards[shard].get(name)
            if info is None:
                raise CheckpointError(f"index maps {name!r} to {shard}, which does not hold it")
            infos.append(info)
        return cls(infos, index_path)

    def names(self) -> tuple[str, ...]:
        return tuple(self._by_name)

    def info(self, name: str) -> TensorInfo:
        try:
            return self._by_name[name]
        except KeyError:
            raise CheckpointError(f"checkpoint has no tensor named {name!r}") from None

    def __contains__(self, name: str) -> bool:
        return name in self._by_name

    def get_tensors(self, names: Iterable[str] | None = None) -> dict[str, torch.Tensor]:
        """Copies of the named tensors (all of them by default), in host memory."""

        wanted = self.names() if names is None else tuple(names)
        return read_tensors(self.info(name) for name in wanted)

    def view(self) -> TensorView:
        """The tensors by name, each mapped from its file when it is asked for and
        dropped when the caller lets go of it (mini_llm/checkpoint.py:62-68: payloads
        stay unmapped until needed).  This is what the model is loaded from."""

        return TensorView(self.names(), lambda name: map_tensor(self.info(name)))


def validate_manifest(
    checkpoint: Checkpoint, expected: Mapping[str, TensorSpec], *, architecture: str, torch_dtype: str | None = None,
) -> None:
    """Raise one ``CheckpointValidationError`` listing every missing tensor,
    every unexpected tensor, every wrong shape and every wrong storage type.

    ``torch_dtype`` (config.json's): every floating tensor must be stored in exactly
    that type, as the reference demands (mini_llm/checkpoint.py:290, 478-481), so a
    mislabelled or mixed-precision checkpoint does not load silently.  ``None`` accepts
    any floating storage type (it is converted at placement)."""

    actual = {info.name: info for info in checkpoint.manifest}
    errors: list[str] = []
    missing = sorted(n for n, spec in expected.items() if n not in actual and not spec.optional)
    unexpected = sorted(actual.keys() - expected.keys())
    if missing:
        errors.append("missing tensors: " + ", ".join(missing))
    if unexpected:
        errors.append("unexpected tensors: " + ", ".join(unexpected))
    for name in sorted(expected.keys() & actual.keys()):
        spec, info = expected[name], actual[name]
        if info.shape != tuple(spec.shape):
            errors.append(
                f"shape mismatch for {name}: expected {tuple(spec.shape)}, got {info.shape}"
            )
        allowed = FLOAT_DTYPES if spec.kind == "float" else INT_DTYPES
        if spec.kind == "float" and torch_dtype is not None:
            allowed = (STORAGE_NAME[torch_dtype],)
        if info.dtype not in allowed:
            errors.append(
                f"dtype mismatch for {name}: expected one of {'/'.join(allowed)}, got {info.dtype}"
            )
    if errors:
        details = "\n  - ".join(errors)
        raise CheckpointValidationError(
            f"checkpoint does not match {architecture} configuration:\n  - {details}"
        )
