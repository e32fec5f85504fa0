"""Token embedding and output head."""

from __future__ import annotations

from typing import Any, Mapping

import torch

from ..ops import functional as F
from ..weights.checkpoint import TensorSpec
from .base import EMBEDDINGS, HEADS, Part, Runtime, WeightedRows
from .linear import Projection


@EMBEDDINGS.register("token_embedding")
class TokenEmbedding(Part):
    """``h = E[token] * scale`` (mini_llm/model/base.py:72-74; Qwen3 uses scale 1)."""

    graph_safe = True

    def __init__(self, *, vocab_size: int, hidden_size: int, scale: float = 1.0) -> None:
        self.vocab_size, self.hidden_size, self.scale = vocab_size, hidden_size, float(scale)
        self.weight: torch.Tensor | None = None

    def tensor_specs(self) -> dict[str, TensorSpec]:
        return {"weight": TensorSpec((self.vocab_size, self.hidden_size))}

    def load(self, tensors: Mapping[str, torch.Tensor], runtime: Runtime) -> None:
        self.runtime = runtime
        self.weight = runtime.place_matrix(tensors["weight"])

    fuses_norms = True    # takes a keyword ``next_norm`` and may return (rows, WeightedRows for that norm)

    def forward(self, token_ids: torch.Tensor, next_norm: Any = None):
        fusable = next_norm.fusable() if next_norm is not None and Projection.FUSE_NORMS else None
        if (fusable is not None and self.runtime.dtype == torch.bfloat16 and token_ids.shape[0] <= 16
                and fusable[0].shape[0] == self.hidden_size and self.hidden_size % 8 == 0 and self.hidden_size <= 8 * 2048):
            rows, weighted, row_scale = F.embedding_weighted(token_ids, self.weight, self.scale, *fusable)
            return rows, WeightedRows(weighted, row_scale)
        return F.embedding(token_ids, self.weight, self.scale)


@HEADS.register("linear_head")
class OutputHead(Part):
    """``logits = h W^T`` in float32, no bias (mini_llm/model/qwen.py:112).  With
    ``tied`` the weight may be absent from the checkpoint; the embedding matrix
    is used then.  A stored ``lm_head.weight`` is always used when present."""

    graph_safe = True

    def __init__(self, *, vocab_size: int, hidden_size: int, tied: bool = False) -> None:
        self.vocab_size, self.hidden_size, self.tied = vocab_size, hidden_size, bool(tied)

    def tensor_specs(self) -> dict[str, TensorSpec]:
        return {"weight": TensorSpec((self.vocab_size, self.hidden_size), optional=self.tied)}

    def load(self, tensors: Mapping[str, torch.Tensor], runtime: Runtime, *, embedding: TokenEmbedding | None = None) -> None:
        self.runtime = runtime
        if "weight" in tensors:
            self.proj = Projection([tensors["weight"]], None, runtime)
        elif self.tied and embedding is not None:
            self.proj = Projection.__new__(Projection)
            self.proj.runtime, self.proj.weight, self.proj.bias = runtime, embedding.weight, None
            self.proj.out_features, self.proj.in_features = embedding.weight.shape
        else:
            raise KeyError("output head has no weight and is not tied to the embedding")

    fuses_norms = True    # takes ``WeightedRows`` prepared for the final norm

    def forward(self, x: "torch.Tensor | WeightedRows") -> torch.Tensor:
        return self.proj(x, torch.float32)
