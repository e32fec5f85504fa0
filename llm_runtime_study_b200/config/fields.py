"""Typed readers for ``config.json`` values.

Same discipline as the reference's ``_required`` (mini_llm/config.py:26-42): a
missing key and a value of the wrong JSON type are both errors, and a boolean is
never accepted where an integer is expected (``True`` is an ``int`` in Python).
"""

from __future__ import annotations

import json
from pathlib import Path
from typing import Any, Mapping

from ..errors import ConfigError

_MISSING = object()


def _type_name(expected: type | tuple[type, ...]) -> str:
    types = expected if isinstance(expected, tuple) else (expected,)
    return " or ".join(t.__name__ for t in types)


def _check(name: str, value: Any, expected: type | tuple[type, ...]) -> Any:
    types = expected if isinstance(expected, tuple) else (expected,)
    if not isinstance(value, types) or (isinstance(value, bool) and bool not in types):
        raise ConfigError(
            f"{name} must be {_type_name(expected)}, got {type(value).__name__}"
        )
    return value


def required(raw: Mapping[str, Any], name: str, expected: type | tuple[type, ...]) -> Any:
    """Return ``raw[name]`` after checking presence and JSON type."""

    if name not in raw:
        raise ConfigError(f"missing required configuration field: {name}")
    return _check(name, raw[name], expected)


def optional(
    raw: Mapping[str, Any], name: str, expected: type | tuple[type, ...], default: Any
) -> Any:
    """Return ``raw[name]`` (type-checked) or ``default`` when the key is absent."""

    value = raw.get(name, _MISSING)
    if value is _MISSING:
        return default
    return _check(name, value, expected)


def token_id_tuple(raw: Mapping[str, Any], name: str) -> tuple[int, ...]:
    """An integer or a non-empty list of integers (mini_llm/config.py:126-134)."""

    value = raw.get(name)
    if isinstance(value, int) and not isinstance(value, bool):
        return (value,)
    if (
        isinstance(value, list)
        and value
        and all(isinstance(v, int) and not isinstance(v, bool) for v in value)
    ):
        return tuple(value)
    raise ConfigError(f"{name} must be an integer or a non-empty integer list")


def read_config_dict(model_dir: str | Path) -> dict[str, Any]:
    """Read ``config.json`` of a model folder (mini_llm/config.py:108-123)."""

    model_path = Path(model_dir)
    config_path = model_path / "config.json"
    if not model_path.is_dir():
        raise ConfigError(f"model directory does not exist: {model_path}")
    if not config_path.is_file():
        raise ConfigError(f"model configuration does not exist: {config_path}")
    try:
        raw = json.loads(config_path.read_text(encoding="utf-8"))
    except json.JSONDecodeError as exc:
        raise ConfigError(f"invalid JSON in {config_path}: {exc}") from exc
    if not isinstance(raw, dict):
        raise ConfigError(f"configuration root must be an object: {config_path}")
    return raw
