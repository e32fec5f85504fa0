"""Gated feed-forward (SwiGLU)."""

from __future__ import annotations

from typing import Any, Mapping

import torch

from ..ops import functional as F
from ..weights.checkpoint import TensorSpec
from .base import FEED_FORWARDS, FeedForward, Runtime
from .linear import Projection


@FEED_FORWARDS.register("swiglu")
class SwiGLU(FeedForward):
    """``down(silu(gate(x)) * up(x))`` without biases (mini_llm/nn/mlp.py:80-87).
    gate and up are one stacked product; the activation and the product with
    ``up`` are computed in float32 and rounded once."""

    graph_safe = True

    def __init__(self, *, hidden_size: int, intermediate_size: int) -> None:
        if hidden_size <= 0 or intermediate_size <= 0:
            raise ValueError("swiglu sizes must be positive")
        self.hidden_size, self.intermediate_size = hidden_size, intermediate_size

    def tensor_specs(self) -> dict[str, TensorSpec]:
        h, i = self.hidden_size, self.intermediate_size
        return {
            "gate_proj.weight": TensorSpec((i, h)),
            "up_proj.weight": TensorSpec((i, h)),
            "down_proj.weight": TensorSpec((h, i)),
        }

    def load(self, tensors: Mapping[str, torch.Tensor], runtime: Runtime) -> None:
        self.runtime = runtime
        gate, up = runtime.place_matrix(tensors["gate_proj.weight"]), runtime.place_matrix(tensors["up_proj.weight"])
        # When the width allows, gate and up rows are interleaved in blocks of eight
        # ([g0..g7, u0..u7, g8..g15, ...]): a projection kernel then holds matching gate and
        # up features in one tile and can apply SiLU * up before it writes anything.
        self.interleaved = self.intermediate_size % 8 == 0
        if self.interleaved:
            blocks = self.intermediate_size // 8
            stacked = torch.stack((gate.view(blocks, 8, -1), up.view(blocks, 8, -1)), dim=1).reshape(2 * self.intermediate_size, -1)
            del gate, up
            self.gate_up_proj = Projection([stacked], None, runtime)
            del stacked
        else:
            self.gate_up_proj = Projection([gate, up], None, runtime)
        self.down_proj = Projection([tensors["down_proj.weight"]], None, runtime)

    adds_to_residual = True
    fuses_norms = True

    def forward(self, x: Any, ctx: Any, residual: torch.Tensor | None = None, next_norm: Any = None):
        hidden = self.gate_up_proj.swiglu(x) if self.interleaved else F.silu_mul(self.gate_up_proj(x))
        return self.down_proj(hidden, torch.float32, add_to=residual, next_norm=next_norm)
