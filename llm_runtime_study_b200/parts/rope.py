"""Rotary position encoding (half-split convention)."""

from __future__ import annotations

from typing import Mapping

import torch

from .base import POSITION_ENCODINGS, PositionEncoding, Runtime


@POSITION_ENCODINGS.register("rope")
class RotaryEmbedding(PositionEncoding):
    """``inv_freq[i] = 1 / theta^(2i / rotary_dim)``, built in float32 on the host
    with the same expression as the reference (mini_llm/nn/rope.py:37-40); the
    angle ``float32(position) * inv_freq[i]`` and its sine and cosine are formed
    in float32 inside the fused kernel (mini_llm/nn/rope.py:74-80).  Pairs are
    ``(i, i + rotary_dim/2)`` (mini_llm/nn/rope.py:110-114).  ``rotary_dim``
    smaller than the head size leaves the remaining columns unrotated."""

    graph_safe = True

    def __init__(self, head_dim: int, theta: float, rotary_dim: int | None = None) -> None:
        rotary_dim = head_dim if rotary_dim is None else rotary_dim
        if head_dim <= 0 or rotary_dim <= 0 or rotary_dim % 2 or rotary_dim > head_dim:
            raise ValueError(f"rope needs an even rotary_dim in (0, head_dim], got {rotary_dim}, {head_dim}")
        if theta <= 0:
            raise ValueError(f"rope theta must be positive, got {theta}")
        self.head_dim, self.theta, self.rotary_dim = head_dim, float(theta), rotary_dim
        self.inv_freq: torch.Tensor | None = None

    def load(self, tensors: Mapping[str, torch.Tensor], runtime: Runtime) -> None:
        self.runtime = runtime
        dims = torch.arange(0, self.rotary_dim, 2, dtype=torch.float32)
        self.inv_freq = (1.0 / (self.theta ** (dims / self.rotary_dim))).to(runtime.device)

    def rotary_parameters(self) -> tuple[torch.Tensor, int]:
        return self.inv_freq, self.rotary_dim
