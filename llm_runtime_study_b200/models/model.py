"""The generic decoder: embedding, the layers in their given order, the final
norm and the output head on the rows whose logits are wanted
(mini_llm/model/base.py:55-89 for the traversal)."""

from __future__ import annotations

from typing import Any, Mapping

import torch

from ..cache.manager import CacheLayout, CacheManager, LayerCache
from ..parts.base import ResidualStream, Runtime
from ..weights.checkpoint import TensorSpec
from ..weights.view import TensorView
from .description import ModelDescription, build_parts


class DecoderModel:
    def __init__(self, description: ModelDescription) -> None:
        self.description = description
        parts = build_parts(description)
        self.embedding_prefix, self.embedding = parts["embedding"]
        self.blocks = parts["blocks"]  # [(prefix, block)]
        self.final_norm_prefix, self.final_norm = parts["final_norm"]
        self.head_prefix, self.head = parts["head"]
        self.order = description.order
        self.runtime: Runtime | None = None
        self._layer_caches: list[LayerCache] | None = None

    # ------------------------------------------------------------ weights
    def tensor_schema(self) -> dict[str, TensorSpec]:
        schema: dict[str, TensorSpec] = {}
        named = [(self.embedding_prefix, self.embedding), *self.blocks,
                 (self.final_norm_prefix, self.final_norm), (self.head_prefix, self.head)]
        for prefix, part in named:
            for name, spec in part.tensor_specs().items():
                schema[f"{prefix}.{name}"] = spec
        return schema

    def load(self, tensors: Mapping[str, torch.Tensor], runtime: Runtime) -> None:
        """Place every weight.  ``tensors`` is keyed by checkpoint name and has
        been validated against ``tensor_schema()`` already."""

        self.runtime = runtime
        view = TensorView.of(tensors)
        self.embedding.load(view.sub(self.embedding_prefix), runtime)
        for prefix, block in self.blocks:
            block.load(view.sub(prefix), runtime)
        self.final_norm.load(view.sub(self.final_norm_prefix), runtime)
        self.head.load(view.sub(self.head_prefix), runtime, embedding=self.embedding)

    # -------------------------------------------------------------- cache
    def cache_layout(self) -> CacheLayout:
        """One requirement per *run* of a layer (a layer named twice in the order
        has two caches); a run that uses an earlier run's cache asks for none."""

        needs = []
        for layer_index, source in zip(self.order, self.description.cache_of):
            needs.append(None if source is not None else self.blocks[layer_index][1].mixer.cache_requirement())
        return CacheLayout.from_requirements(needs)

    def bind_cache(self, manager: CacheManager) -> None:
        self._layer_caches = [
            manager.layer_cache(run if source is None else source)
            for run, source in enumerate(self.description.cache_of)
        ]

    def graph_safe(self) -> bool:
        """Whether every part allows its launches to be replayed from a CUDA graph."""

        parts = [self.embedding, *(block for _, block in self.blocks), self.final_norm, self.head]
        return all(part.capture_safe() for part in parts)

    # ------------------------------------------------------------ forward
    def forward(self, ctx: Any) -> torch.Tensor | None:
        """Run the batch in ``ctx``; return float32 logits ``[wanted, vocab]``
        (``None`` when no row is wanted: the cache is written all the same)."""

        blocks = [self.blocks[index][1] for index in self.order]
        # the norm that reads the stream after each block: the next block's first norm, at last the final norm
        readers = [block.first_norm() for block in blocks[1:]] + [self.final_norm]
        if getattr(self.embedding, "fuses_norms", False):
            first = self.embedding.forward(ctx.token_ids, next_norm=blocks[0].first_norm())
        else:
            first = self.embedding.forward(ctx.token_ids)
        if isinstance(first, tuple):     # (rows, the same rows prepared for the first norm)
            stream = ResidualStream(first[0], weighted=first[1], weighted_for=blocks[0].first_norm())
        else:
            stream = ResidualStream(first)
        for run, (block, reader) in enumerate(zip(blocks, readers)):
            if block.fuses_norms:
                block.forward(stream, ctx, self._layer_caches[run], next_norm=reader)
            else:
                block.forward(stream, ctx, self._layer_caches[run])
        if ctx.num_logit_rows == 0:
            return None
        if stream.weighted is not None and stream.weighted_for is self.final_norm and getattr(ctx, "logits_at_every_row", False):
            x = stream.take_rows(self.final_norm, self.head)       # every row is wanted, in order: no gather
        else:
            x = self.final_norm.norm_rows(stream.resid, stream.delta, ctx.logit_rows)
        return self.head.forward(x)
