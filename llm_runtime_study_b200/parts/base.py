"""Interfaces and registries of the parts a model is put together from.

A model is data: a list of layer descriptions, each naming the *kind* of its
mixer, feed-forward, norms and position encoding together with their sizes and
constants, plus the order in which the layers run.  A kind is a class
registered here under a name.  No part knows which model it is in: it sees its
own parameters, its own weights (by names relative to its prefix), and the
``StepContext`` of the batch being run.

Interfaces (all tensors live on the CUDA device; ``x`` is ``[tokens, width]``):

``Part``            ``tensor_specs() -> {relative name: TensorSpec}``;
                    ``load(tensors, runtime)`` places weights (fusing if it wants).
``Norm``            ``add_norm(resid, delta, ctx) -> x`` adds ``delta`` into the
                    float32 residual stream in place and returns the normalised rows
                    in the activation type; ``norm_rows(resid, rows) -> x`` gathers.
``PositionEncoding````rotary_parameters()`` returns ``(inv_freq, rotary_dim)`` for the
                    fused rotate-and-write kernel, or ``None``; then
                    ``apply(q, k, ctx)`` is called on ``[tokens, heads, d]`` instead.
``Mixer``           ``cache_requirement()`` says what per-request memory it needs
                    (``PagedKV``, ``FixedState`` or ``None``);
                    ``forward(x, ctx, cache) -> float32 [tokens, hidden]``.
``FeedForward``     ``forward(x, ctx) -> float32 [tokens, hidden]``.
``Block``           ``forward(stream, ctx, cache)`` where ``stream`` carries the
                    residual rows and the not-yet-added output of the previous part.
Embeddings (``forward(token_ids) -> float32 [tokens, hidden]``) and output heads
(``forward(x) -> float32 [rows, vocab]``; ``load`` also gets ``embedding=`` for tied
weights) are registered kinds too.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Mapping

import torch

from ..errors import RegistryError
from ..weights.checkpoint import TensorSpec


# ---------------------------------------------------------------- runtime
@dataclass(frozen=True)
class Runtime:
    """Where and in which type a model runs.  ``dtype`` is the storage type of
    matrices, activations and the cache: ``torch.bfloat16`` (serving) or
    ``torch.float32`` (verification; FFMA only, no reduced-precision matrix mode)."""

    device: torch.device
    dtype: torch.dtype

    def place_matrix(self, t: torch.Tensor) -> torch.Tensor:
        """To the device as stored (for a mapped file: straight from its pages), then to the run type there."""

        return t.to(device=self.device).to(dtype=self.dtype).contiguous()

    def place_vector_f32(self, t: torch.Tensor) -> torch.Tensor:
        """Norm weights and other small vectors are kept in float32 in both modes."""

        return t.to(device=self.device).to(dtype=torch.float32).contiguous()


# ------------------------------------------------------- cache requirements
@dataclass(frozen=True)
class PagedKV:
    """Keys and values that grow with the sequence, kept in pages.  ``window``
    (tokens) bounds how far back the mixer reads; pages wholly behind it are
    given back early.  Layers with equal requirements share a group of pages."""

    num_kv_heads: int
    head_dim: int
    window: int | None = None


@dataclass(frozen=True)
class FixedState:
    """Per-request state of fixed size: one array ``[slots, *shape]`` per layer,
    zeroed when a request takes a slot."""

    shape: tuple[int, ...]
    dtype: torch.dtype = torch.float32


# ------------------------------------------------------------------ parts
class Part:
    """Anything that owns weights."""

    # Whether the part's launches may be recorded into a CUDA graph and replayed for other batches
    # of the same size.  Such a part takes everything that changes from step to step out of device
    # tensors of the context (``ctx.slots``, ``ctx.positions``, ``ctx.kv_len``, the block tables),
    # never out of its host-side lists (under capture ``ctx.entry_slots`` is ``None`` and
    # ``ctx.kv_lens`` holds upper bounds), launches the same kernels whatever the data, and lets rows
    # that pad the batch (slot ``manager.padding_slot``, length 0) write only into that slot's row of
    # its state.  The kinds of this package do; a kind registered from outside must say so itself.
    graph_safe = False

    def children(self) -> tuple["Part", ...]:
        """The parts this part is made of (their weights live under its prefix)."""

        return ()

    def capture_safe(self) -> bool:
        return bool(self.graph_safe) and all(child.capture_safe() for child in self.children())

    def tensor_specs(self) -> dict[str, TensorSpec]:
        return {}

    def load(self, tensors: Mapping[str, torch.Tensor], runtime: Runtime) -> None:
        self.runtime = runtime


class Norm(Part):
    def add_norm(self, resid: torch.Tensor, delta: torch.Tensor | None) -> torch.Tensor:
        raise NotImplementedError

    def norm_rows(self, resid: torch.Tensor, delta: torch.Tensor | None, rows: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError


class PositionEncoding(Part):
    def rotary_parameters(self) -> tuple[torch.Tensor, int] | None:
        return None

    def apply(self, q: torch.Tensor, k: torch.Tensor | None, ctx: Any) -> None:
        """Rotate/shift ``q`` and ``k`` in place (only called when
        ``rotary_parameters()`` is ``None``)."""


class Mixer(Part):
    # A part that sets this takes a keyword ``residual`` (the float32 residual rows, already
    # holding everything before this part) and may add its output to them in place, returning
    # ``None`` instead of the output; the block then has nothing left to add.
    adds_to_residual = False

    def cache_requirement(self) -> PagedKV | FixedState | None:
        return None

    def forward(self, x: torch.Tensor, ctx: Any, cache: Any) -> torch.Tensor:
        raise NotImplementedError


class FeedForward(Part):
    adds_to_residual = False    # as for Mixer

    def forward(self, x: torch.Tensor, ctx: Any) -> torch.Tensor:
        raise NotImplementedError


class Block(Part):
    mixer: Mixer

    def forward(self, stream: "ResidualStream", ctx: Any, cache: Any) -> None:
        raise NotImplementedError


@dataclass
class ResidualStream:
    """The float32 residual rows and the output of the last part that has not
    been added yet: the next norm adds it while it normalises (one pass over
    memory instead of two)."""

    resid: torch.Tensor
    delta: torch.Tensor | None = None


# --------------------------------------------------------------- registries
class Registry:
    def __init__(self, what: str) -> None:
        self.what = what
        self._kinds: dict[str, Callable[..., Any]] = {}

    def register(self, kind: str, factory: Callable[..., Any] | None = None, *, replace: bool = False):
        def _add(f):
            if kind in self._kinds and not replace:
                raise RegistryError(f"{self.what} kind {kind!r} is already registered")
            self._kinds[kind] = f
            return f

        return _add if factory is None else _add(factory)

    def build(self, description: Mapping[str, Any]) -> Any:
        """``description`` is ``{"kind": name, **parameters}``."""

        params = dict(description)
        kind = params.pop("kind", None)
        if kind not in self._kinds:
            known = ", ".join(sorted(self._kinds))
            raise RegistryError(f"unknown {self.what} kind {kind!r}; registered: {known}")
        return self._kinds[kind](**params)

    def kinds(self) -> tuple[str, ...]:
        return tuple(sorted(self._kinds))


EMBEDDINGS = Registry("embedding")
HEADS = Registry("output head")
NORMS = Registry("norm")
POSITION_ENCODINGS = Registry("position encoding")
MIXERS = Registry("mixer")
FEED_FORWARDS = Registry("feed-forward")
BLOCKS = Registry("block")
