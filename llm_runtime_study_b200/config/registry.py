"""One registry from an architecture's name to everything built from it.

The reference keeps three parallel dicts keyed by ``model_type``: the model
class (mini_llm/model/loader.py:13-33), the checkpoint schema builder
(mini_llm/checkpoint.py:389-405) and the config class (mini_llm/config.py:501-512).
Here one entry carries all three, so adding an architecture is one
``register_architecture`` call.
"""

from __future__ import annotations

from dataclasses import dataclass
from pathlib import Path
from typing import Any, Callable, Mapping

from ..errors import ConfigError
from .fields import read_config_dict


@dataclass(frozen=True)
class Architecture:
    """What an architecture contributes.

    ``config_from_dict(raw)`` returns its typed configuration.
    ``describe(config)`` returns a ``ModelDescription`` (the list of layer
    descriptions, the order in which they run, and the embedding/head/norm
    descriptions) from which the generic model is built; it names part kinds
    only, never sizes of its own.
    """

    name: str
    model_type: str
    config_from_dict: Callable[[Mapping[str, Any]], Any]
    describe: Callable[[Any], Any]


_BY_NAME: dict[str, Architecture] = {}
_BY_MODEL_TYPE: dict[str, Architecture] = {}


def register_architecture(arch: Architecture, *, replace: bool = False) -> None:
    if not replace and (arch.name in _BY_NAME or arch.model_type in _BY_MODEL_TYPE):
        raise ConfigError(f"architecture {arch.name!r} / {arch.model_type!r} already registered")
    _BY_NAME[arch.name] = arch
    _BY_MODEL_TYPE[arch.model_type] = arch


def registered_architectures() -> tuple[str, ...]:
    return tuple(sorted(_BY_NAME))


def architecture_for(raw: Mapping[str, Any]) -> Architecture:
    """Pick the entry by ``model_type`` (as the reference does), else by
    ``architectures[0]``."""

    model_type = raw.get("model_type")
    if isinstance(model_type, str) and model_type in _BY_MODEL_TYPE:
        return _BY_MODEL_TYPE[model_type]
    names = raw.get("architectures")
    if isinstance(names, list) and names and isinstance(names[0], str) and names[0] in _BY_NAME:
        return _BY_NAME[names[0]]
    if "model_type" not in raw:
        raise ConfigError("missing required configuration field: model_type")
    supported = ", ".join(sorted(_BY_MODEL_TYPE))
    raise ConfigError(f"unsupported model_type {model_type!r}; expected one of: {supported}")


def load_config(model_dir: str | Path) -> tuple[Architecture, Any]:
    """Read ``config.json`` and return ``(architecture entry, typed config)``."""

    raw = read_config_dict(model_dir)
    arch = architecture_for(raw)
    return arch, arch.config_from_dict(raw)
