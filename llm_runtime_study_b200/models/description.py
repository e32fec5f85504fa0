"""A model as data: which parts, with which sizes, in which order.

An architecture's ``describe(config)`` returns a ``ModelDescription``.  The
generic ``DecoderModel`` is built from it; the tensor schema, the cache groups
and the random-weights mode are derived from it.  The order in which layers run
is a list too: it may name a layer twice (weights shared between depths; each
run of a layer has a cache of its own), and a run may instead use the cache that
an earlier run writes (``cache_of``).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping

from ..parts import embedding as _embedding_kinds  # noqa: F401  (registers the embedding and head kinds of this package)
from ..parts.base import BLOCKS, EMBEDDINGS, HEADS, NORMS
from ..weights.checkpoint import TensorSpec


@dataclass(frozen=True)
class LayerDescription:
    """One layer: ``block`` is ``{"kind": ..., "mixer": {...}, "feed_forward": {...},
    ...}`` for the block registry; ``prefix`` is where its tensors live in the
    checkpoint."""

    block: Mapping[str, Any]
    prefix: str


@dataclass(frozen=True)
class ModelDescription:
    architecture: str
    vocab_size: int
    hidden_size: int
    max_positions: int
    eos_token_ids: tuple[int, ...]
    embedding: Mapping[str, Any]          # embedding description ("kind", default "token_embedding") + "prefix"
    layers: tuple[LayerDescription, ...]
    order: tuple[int, ...]                # indices into ``layers``, in execution order
    final_norm: Mapping[str, Any]         # norm description + "prefix"
    head: Mapping[str, Any]               # output head description ("kind", default "linear_head") + "prefix"
    cache_of: tuple[int | None, ...] = () # per run: the earlier run whose cache it uses (None: its own)
    extra: Mapping[str, Any] = field(default_factory=dict)

    def __post_init__(self) -> None:
        n = len(self.layers)
        if not self.order or any(not 0 <= i < n for i in self.order):
            raise ValueError(f"layer order {self.order} does not index {n} layers")
        if not self.cache_of:
            object.__setattr__(self, "cache_of", (None,) * len(self.order))
        if len(self.cache_of) != len(self.order):
            raise ValueError("cache_of needs one entry for every run in order")
        for run, src in enumerate(self.cache_of):
            if src is not None and (not 0 <= src < run or self.cache_of[src] is not None):
                raise ValueError(f"run {run} uses the cache of run {src}, which is not an earlier run with a cache of its own")


def _split(description: Mapping[str, Any]) -> tuple[str, dict[str, Any]]:
    params = dict(description)
    return params.pop("prefix"), params


def build_parts(description: ModelDescription):
    """Instantiate every part (no weights yet)."""

    emb_prefix, emb_params = _split(description.embedding)
    norm_prefix, norm_params = _split(description.final_norm)
    head_prefix, head_params = _split(description.head)
    return {
        "embedding": (emb_prefix, EMBEDDINGS.build({"kind": "token_embedding", **emb_params})),
        "blocks": [(layer.prefix, BLOCKS.build(layer.block)) for layer in description.layers],
        "final_norm": (norm_prefix, NORMS.build(norm_params)),
        "head": (head_prefix, HEADS.build({"kind": "linear_head", **head_params})),
    }


def tensor_schema(description: ModelDescription) -> dict[str, TensorSpec]:
    """Every tensor the checkpoint must (or may) hold, by its full name."""

    parts = build_parts(description)
    schema: dict[str, TensorSpec] = {}
    for prefix, part in (parts["embedding"], *parts["blocks"], parts["final_norm"], parts["head"]):
        for name, spec in part.tensor_specs().items():
            schema[f"{prefix}.{name}"] = spec
    return schema
