"""bfloat16 tensor-core attention kernels (built per head size)."""

from __future__ import annotations

from typing import Any

import torch


def try_paged_attention(q: torch.Tensor, cache: Any, ctx: Any, table: torch.Tensor, *, scale: float, window: int):
    """Return the attention output, or ``None`` when no tensor-core kernel takes
    this case (the caller then uses the CUDA-core kernel)."""

    return None


def build(head_dim: int) -> None:
    """Compile the kernels for one head size (no-op until they exist)."""
