"""A read-only, prefix-addressable view of named tensors.

Parts ask for their tensors by names relative to their own prefix.  The view
resolves a name on demand, so the source can be a dict of loaded tensors or a
generator that draws a random tensor only when it is asked for (at real sizes
that keeps a single layer's temporaries alive instead of the whole model's).
"""

from __future__ import annotations

from typing import Callable, Iterable, Mapping

import torch


class TensorView:
    def __init__(self, names: Iterable[str], get: Callable[[str], torch.Tensor], prefix: str = "") -> None:
        self._names = frozenset(names)
        self._get = get
        self._prefix = prefix

    @classmethod
    def of(cls, tensors: "Mapping[str, torch.Tensor] | TensorView") -> "TensorView":
        if isinstance(tensors, TensorView):
            return tensors
        return cls(tensors.keys(), tensors.__getitem__)

    def sub(self, prefix: str) -> "TensorView":
        return TensorView(self._names, self._get, f"{self._prefix}{prefix}.")

    def __contains__(self, name: str) -> bool:
        return f"{self._prefix}{name}" in self._names

    def __getitem__(self, name: str) -> torch.Tensor:
        full = f"{self._prefix}{name}"
        if full not in self._names:
            raise KeyError(full)
        return self._get(full)

    def keys(self) -> list[str]:
        cut = len(self._prefix)
        return sorted(n[cut:] for n in self._names if n.startswith(self._prefix))
