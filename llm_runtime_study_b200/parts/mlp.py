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
        self.gate_up_proj = Projection([tensors["gate_proj.weight"], tensors["up_proj.weight"]], None, runtime)
        self.down_proj = Projection([tensors["down_proj.weight"]], None, runtime)

    def forward(self, x: torch.Tensor, ctx: Any) -> torch.Tensor:
        return self.down_proj(F.silu_mul(self.gate_up_proj(x)), torch.float32)
