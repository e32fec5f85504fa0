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
class PagedTensors:
    """Per-token memory that grows with the sequence, kept in pages: what a mixer asks the cache for.
    ``tensors`` names each tensor and gives its shape per token; a tensor of per-token shape ``(a, b, ...)``
    is held as ``[pages, a, page_size, b, ...]`` (one (page, a) tile is contiguous), one of shape ``(a,)`` as
    ``[pages, page_size, a]``.  ``window`` (tokens) bounds how far back the mixer reads; pages wholly behind
    it are given back early and the group's pool is sized for the window rather than for whole sequences.
    ``page_size`` is the group's own (``None``: the cache manager's default).  Layers with equal
    requirements share a group of pages: one page id addresses the same positions in each of them."""

    tensors: tuple[tuple[str, tuple[int, ...]], ...]
    window: int | None = None
    page_size: int | None = None


@dataclass(frozen=True)
class PagedKV(PagedTensors):
    """Keys and values of ``num_kv_heads`` heads of ``head_dim`` each: the request of an attention mixer."""

    num_kv_heads: int = 0
    head_dim: int = 0

    def __init__(self, num_kv_heads: int, head_dim: int, window: int | None = None, page_size: int | None = None) -> None:
        object.__setattr__(self, "tensors", (("keys", (num_kv_heads, head_dim)), ("values", (num_kv_heads, head_dim))))
        object.__setattr__(self, "window", window)
        object.__setattr__(self, "page_size", page_size)
        object.__setattr__(self, "num_kv_heads", num_kv_heads)
        object.__setattr__(self, "head_dim", head_dim)


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
    def fusable(self) -> tuple[torch.Tensor, float] | None:
        """(weight, eps) if the norm is ``weight * x * rsqrt(mean(x^2) + eps)``, which a projection before it
        and one after it can carry out between them (see ``WeightedRows``); ``None`` for any other norm."""

        return None

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
    # A part that sets this as well takes ``WeightedRows`` as its input where it would take normalised
    # rows, and a keyword ``next_norm`` (the norm that follows it, or ``None``): when it adds into the
    # residual rows it may return ``WeightedRows`` prepared for that norm instead of ``None``.
    fuses_norms = False

    def cache_requirement(self) -> PagedKV | FixedState | None:
        return None

    def forward(self, x: torch.Tensor, ctx: Any, cache: Any) -> torch.Tensor:
        raise NotImplementedError


class FeedForward(Part):
    adds_to_residual = False    # as for Mixer
    fuses_norms = False         # as for Mixer

    def forward(self, x: torch.Tensor, ctx: Any) -> torch.Tensor:
        raise NotImplementedError


class Block(Part):
    mixer: Mixer
    # A block that sets this takes a keyword ``next_norm``: the norm that will read the stream after
    # this block (the next block's first norm, or the model's final norm), so that its last part may
    # prepare the rows for it.
    fuses_norms = False

    def first_norm(self) -> "Norm | None":
        """The norm that reads the stream first when this block runs, if it has one."""

        return None

    def forward(self, stream: "ResidualStream", ctx: Any, cache: Any) -> None:
        raise NotImplementedError


@dataclass
class WeightedRows:
    """Rows of the residual stream multiplied by a norm's weight and rounded to the activation type,
    still lacking the norm's factor ``rsqrt(mean of squares + eps)``.  That factor is one number per
    row (``scale``) and commutes with a matrix product, so a projection that is handed such rows applies
    it to its results instead (``Projection`` does, where its kernel can).  This is how a part that adds
    its output into the residual rows can do the work of the norm that follows while it has the rows in
    its hands, and a batch of a few decoded tokens runs without norm kernels."""

    values: torch.Tensor        # [rows, width], activation type
    scale: torch.Tensor         # [16] float32; the first ``rows`` entries count

    def normalised(self) -> torch.Tensor:
        """The normalised rows themselves, for a consumer that cannot apply the factor (plain tensor operations)."""

        rows = self.values.shape[0]
        return (self.values.float() * self.scale[:rows, None]).to(self.values.dtype)


@dataclass
class ResidualStream:
    """The float32 residual rows and the output of the last part that has not
    been added yet: the next norm adds it while it normalises (one pass over
    memory instead of two).  ``weighted`` holds, when the last part has added its
    output itself and prepared the rows for the norm ``weighted_for``, those rows."""

    resid: torch.Tensor
    delta: torch.Tensor | None = None
    weighted: WeightedRows | None = None
    weighted_for: Any = None

    def take_rows(self, norm: "Norm", consumer: Any) -> "torch.Tensor | WeightedRows":
        """What ``consumer`` gets as the rows normalised by ``norm``."""

        rows, made_for = self.weighted, self.weighted_for
        self.weighted = self.weighted_for = None
        if rows is not None and made_for is norm:
            return rows if getattr(consumer, "fuses_norms", False) else rows.normalised()
        return norm.add_norm(self.resid, self.delta)

    def put(self, out: "torch.Tensor | WeightedRows | None", norm: "Norm | None") -> None:
        """Record what a part returned: its output (to be added by the next norm), ``None`` (it added its
        output itself), or the rows it prepared for ``norm`` (added, and that norm half done)."""

        self.delta = self.weighted = self.weighted_for = None
        if isinstance(out, WeightedRows):
            self.weighted, self.weighted_for = out, norm
        else:
            self.delta = out


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
