"""Choice of the attention kernel for a batch."""

from __future__ import annotations

from typing import Any

import torch

from . import functional as F


def paged_attention(q: torch.Tensor, cache: Any, ctx: Any, *, scale: float, window: int = 0) -> torch.Tensor:
    """Causal attention of the batch's query tokens over their requests' pages.

    float32 runtime: the CUDA-core kernel whose reduction order depends on the
    token's position only.  bfloat16 runtime: the tensor-core kernels (one for
    batches that hold prompt portions, a split-sequence one for batches of
    single decoded tokens) where they are built for the head size; the CUDA-core
    kernel otherwise.
    """

    table = ctx.block_table(cache.group)
    if q.dtype == torch.bfloat16:
        from . import attention_bf16

        out = attention_bf16.try_paged_attention(q, cache, ctx, table, scale=scale, window=window)
        if out is not None:
            return out
    return F.paged_attention_simt(
        q, cache.keys, cache.values, positions=ctx.positions, token_entry=ctx.token_entry,
        block_table=table, scale=scale, window=window,
    )
