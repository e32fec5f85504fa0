"""The kernels as functions over torch tensors (device memory only).

Activations are ``float32`` or ``bfloat16``; the residual stream, norm weights,
rotary frequencies and logits are always ``float32``.
"""

from __future__ import annotations

import torch

from ..errors import KernelError
from . import native
from .native import call, ptr, require, stream_ptr, tag


def embedding(ids: torch.Tensor, table: torch.Tensor, scale: float = 1.0) -> torch.Tensor:
    """``out[n] = table[ids[n]] * scale`` as float32 (the residual stream's type)."""

    require(ids, "ids", dtype=torch.int32, dims=1)
    require(table, "table", dims=2)
    n, (vocab, hidden) = ids.shape[0], table.shape
    out = torch.empty((n, hidden), dtype=torch.float32, device=table.device)
    call("b200_embedding", ptr(ids), ptr(table), ptr(out), n, hidden, vocab, float(scale),
         tag(table.dtype), stream_ptr())
    return out


def embedding_weighted(ids: torch.Tensor, table: torch.Tensor, scale: float, norm_weight: torch.Tensor, eps: float):
    """For at most 16 tokens: the embedding rows as float32, the same rows times ``norm_weight`` in bfloat16,
    and each row's factor ``rsqrt(mean of squares + eps)`` (``[16]`` floats, what ``gemm_bf16.linear_skinny``
    takes as ``row_scale``).  The row width must be a multiple of a 16-byte vector of the table's type."""

    require(ids, "ids", dtype=torch.int32, dims=1)
    require(table, "table", dims=2)
    n, (vocab, hidden) = ids.shape[0], table.shape
    require(norm_weight, "norm_weight", dtype=torch.float32, shape=(hidden,))
    out = torch.empty((n, hidden), dtype=torch.float32, device=table.device)
    weighted = torch.empty((n, hidden), dtype=torch.bfloat16, device=table.device)
    row_scale = torch.empty(16, dtype=torch.float32, device=table.device)
    call("b200_embedding_weighted", ptr(ids), ptr(table), ptr(out), ptr(norm_weight), ptr(weighted), ptr(row_scale), n, hidden,
         vocab, float(scale), float(eps), tag(table.dtype), stream_ptr())
    return out, weighted, row_scale


def add_rmsnorm(
    resid: torch.Tensor, delta: torch.Tensor | None, weight: torch.Tensor, eps: float,
    out_dtype: torch.dtype, *, rows: torch.Tensor | None = None,
) -> torch.Tensor:
    """``resid += delta`` (in place, float32) and return ``rms_norm(resid) * weight``.

    With ``rows`` the given rows are gathered, normalised and returned, and
    ``resid`` is left as it is (used for the rows whose logits are wanted).
    """

    require(resid, "resid", dtype=torch.float32, dims=2)
    n_src, hidden = resid.shape
    if delta is not None:
        require(delta, "delta", dtype=torch.float32, shape=resid.shape)
    require(weight, "weight", dtype=torch.float32, shape=(hidden,))
    if rows is not None:
        require(rows, "rows", dtype=torch.int32, dims=1)
    n = n_src if rows is None else rows.shape[0]
    out = torch.empty((n, hidden), dtype=out_dtype, device=resid.device)
    call("b200_add_rmsnorm", ptr(resid), ptr(delta), ptr(weight), ptr(out), ptr(rows), n, hidden,
         float(eps), 1 if (rows is None and delta is not None) else 0, tag(out_dtype), stream_ptr())
    return out


def linear_f32(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
    """``x @ weight.T (+ bias)`` in true float32 (FFMA only)."""

    require(x, "x", dtype=torch.float32, dims=2)
    require(weight, "weight", dtype=torch.float32, dims=2)
    m, k = x.shape
    n = weight.shape[0]
    if weight.shape[1] != k:
        raise KernelError(f"linear: x has width {k}, weight expects {weight.shape[1]}")
    if bias is not None:
        require(bias, "bias", dtype=torch.float32, shape=(n,))
    out = torch.empty((m, n), dtype=torch.float32, device=x.device)
    call("b200_gemm_f32", ptr(x), ptr(weight), ptr(bias), ptr(out), m, n, k, k, n, stream_ptr())
    return out


def silu_mul(gate_up: torch.Tensor) -> torch.Tensor:
    """``silu(gate) * up`` for rows laid out as ``[gate | up]``."""

    require(gate_up, "gate_up", dims=2)
    n, two_i = gate_up.shape
    if two_i % 2:
        raise KernelError("silu_mul: row width must be even ([gate | up])")
    out = torch.empty((n, two_i // 2), dtype=gate_up.dtype, device=gate_up.device)
    call("b200_silu_mul", ptr(gate_up), ptr(out), n, two_i // 2, tag(gate_up.dtype), stream_ptr())
    return out


def silu_mul_interleaved(gate_up: torch.Tensor) -> torch.Tensor:
    """``silu(gate) * up`` for rows laid out in blocks of eight, ``[g0..g7 | u0..u7 | g8..g15 | ...]``
    (the layout of a stacked gate/up projection whose kernels can apply the activation themselves)."""

    require(gate_up, "gate_up", dims=2)
    n, two_i = gate_up.shape
    if two_i % 16:
        raise KernelError("silu_mul_interleaved: row width must be a multiple of 16")
    out = torch.empty((n, two_i // 2), dtype=gate_up.dtype, device=gate_up.device)
    call("b200_silu_mul_interleaved", ptr(gate_up), ptr(out), n, two_i // 2, tag(gate_up.dtype), stream_ptr())
    return out


def qk_norm_rope_write(
    qkv: torch.Tensor, *, num_q_heads: int, num_kv_heads: int, head_dim: int,
    q_weight: torch.Tensor | None, k_weight: torch.Tensor | None, eps: float,
    inv_freq: torch.Tensor | None, rotary_dim: int, positions: torch.Tensor,
    token_entry: torch.Tensor, block_table: torch.Tensor | None, page_size: int,
    k_pool: torch.Tensor | None, v_pool: torch.Tensor | None,
) -> torch.Tensor:
    """Per-head RMS norm of q and k (optional), rotary rotation (optional), then q is
    returned as ``[N, nq, d]`` and k, v are written into the paged pools
    ``[pages, nkv, page_size, d]`` at each token's position.  ``num_kv_heads = 0``
    with no pools handles a layer that only reads another layer's cache."""

    require(qkv, "qkv", dims=2)
    n, width = qkv.shape
    if width != (num_q_heads + 2 * num_kv_heads) * head_dim:
        raise KernelError(f"qkv width {width} != (nq + 2 nkv) * d")
    dev, dt = qkv.device, qkv.dtype
    require(positions, "positions", dtype=torch.int32, shape=(n,))
    require(token_entry, "token_entry", dtype=torch.int32, shape=(n,))
    for w, name in ((q_weight, "q_weight"), (k_weight, "k_weight")):
        if w is not None:
            require(w, name, dtype=torch.float32, shape=(head_dim,))
    if inv_freq is not None:
        require(inv_freq, "inv_freq", dtype=torch.float32, shape=(rotary_dim // 2,))
    table_stride = 0
    if num_kv_heads > 0:
        require(block_table, "block_table", dtype=torch.int32, dims=2)
        table_stride = block_table.shape[1]
        for pool, name in ((k_pool, "k_pool"), (v_pool, "v_pool")):
            require(pool, name, dtype=dt, dims=4)
            if tuple(pool.shape[1:]) != (num_kv_heads, page_size, head_dim):
                raise KernelError(f"{name} has shape {tuple(pool.shape)}, expected [pages, {num_kv_heads}, {page_size}, {head_dim}]")
    q_out = torch.empty((n, num_q_heads, head_dim), dtype=dt, device=dev)
    call("b200_qk_norm_rope_write", ptr(qkv), ptr(q_out), ptr(q_weight), ptr(k_weight), float(eps),
         ptr(inv_freq), rotary_dim if inv_freq is not None else 0, ptr(positions), ptr(token_entry),
         ptr(block_table), table_stride, page_size, ptr(k_pool), ptr(v_pool), n, num_q_heads,
         num_kv_heads, head_dim, width, tag(dt), stream_ptr())
    return q_out


def paged_attention_simt(
    q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, *, positions: torch.Tensor,
    token_entry: torch.Tensor, block_table: torch.Tensor, scale: float, window: int = 0,
) -> torch.Tensor:
    """Causal attention of every query token over keys ``0..position`` of its request,
    32-bit arithmetic, reduction order fixed by the token's position alone."""

    require(q, "q", dims=3)
    n, nq, d = q.shape
    require(k_pool, "k_pool", dtype=q.dtype, dims=4)
    require(v_pool, "v_pool", dtype=q.dtype, shape=k_pool.shape)
    _, nkv, page_size, dk = k_pool.shape
    if dk != d:
        raise KernelError(f"q head size {d} != cache head size {dk}")
    if d % 16:
        raise KernelError(f"head size {d} is not a multiple of 16")
    require(positions, "positions", dtype=torch.int32, shape=(n,))
    require(token_entry, "token_entry", dtype=torch.int32, shape=(n,))
    require(block_table, "block_table", dtype=torch.int32, dims=2)
    out = torch.empty_like(q)
    call("b200_paged_attention_simt", ptr(q), ptr(k_pool), ptr(v_pool), ptr(out), ptr(positions),
         ptr(token_entry), ptr(block_table), block_table.shape[1], page_size, n, nq, nkv, d,
         float(scale), int(window), tag(q.dtype), stream_ptr())
    return out
