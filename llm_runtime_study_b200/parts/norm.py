"""RMS normalisation, fused with the residual addition that precedes it."""

from __future__ import annotations

from typing import Mapping

import torch

from ..ops import functional as F
from ..weights.checkpoint import TensorSpec
from .base import NORMS, Norm, Runtime


@NORMS.register("rms_norm")
class RMSNorm(Norm):
    """``y = w * x * rsqrt(mean(x^2) + eps)``: statistics in float32, the weight
    applied as ``w`` (mini_llm/nn/norm.py:42-46).  Random weights are
    ``1 + N(0, 0.05)``."""

    graph_safe = True

    def __init__(self, dim: int, eps: float) -> None:
        if dim <= 0 or eps <= 0:
            raise ValueError(f"rms_norm needs dim > 0 and eps > 0, got {dim}, {eps}")
        self.dim, self.eps = dim, float(eps)
        self.weight: torch.Tensor | None = None

    def tensor_specs(self) -> dict[str, TensorSpec]:
        return {"weight": TensorSpec((self.dim,), init="one_plus_normal", std=0.05)}

    def load(self, tensors: Mapping[str, torch.Tensor], runtime: Runtime) -> None:
        self.runtime = runtime
        self.weight = runtime.place_vector_f32(tensors["weight"])

    def fusable(self) -> tuple[torch.Tensor, float]:
        return self.weight, self.eps

    def add_norm(self, resid: torch.Tensor, delta: torch.Tensor | None) -> torch.Tensor:
        return F.add_rmsnorm(resid, delta, self.weight, self.eps, self.runtime.dtype)

    def norm_rows(self, resid: torch.Tensor, delta: torch.Tensor | None, rows: torch.Tensor) -> torch.Tensor:
        return F.add_rmsnorm(resid, delta, self.weight, self.eps, self.runtime.dtype, rows=rows)
