"""Plain, slow Qwen3 dense forward pass: whole sequences, no cache, CPU.

Written from the reference's formulas; each function cites the file and lines it
restates.  It shares no code with the engine: it takes a ``config.json`` dict
and a ``{tensor name: tensor}`` dict with the checkpoint's own names, and uses
only elementary torch operations (matmul, exp, sum, ...).  ``dtype`` is the
arithmetic type (float32, or float64 to separate rounding from faults).

``store`` (optional) is applied wherever a serving engine with 16-bit activations
keeps a tensor in memory between two operations: the normalised rows, the q/k/v
rows, q and k after the rotation, the attention output, and silu(gate) * up.  With
``store=round_bfloat16`` the plain model carries the same roundings as such an
engine and what is left between the two is the order of the sums; the residual
stream, the statistics and the logits stay in ``dtype`` either way.
"""

from __future__ import annotations

import math
from typing import Mapping

import torch


def _keep(x: torch.Tensor) -> torch.Tensor:
    return x


def round_bfloat16(x: torch.Tensor) -> torch.Tensor:
    """Round to the nearest bfloat16 and widen again."""

    return x.to(torch.bfloat16).to(x.dtype)


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """y = w * x / sqrt(mean(x^2) + eps) over the last axis; the weight is applied
    as ``w``, not ``1 + w`` (mini_llm/nn/norm.py:42-46)."""

    mean_square = (x * x).sum(dim=-1, keepdim=True) / x.shape[-1]
    return weight * (x / torch.sqrt(mean_square + eps))


def rotary_tables(positions: torch.Tensor, head_dim: int, theta: float, dtype: torch.dtype):
    """inv_f[i] = 1 / theta^(2i/d) in float32, angle = float32(p) * inv_f, both halves
    share the angles (mini_llm/nn/rope.py:37-40, 74-80).  Angles are formed in
    float32 exactly as the reference does, then widened to ``dtype``."""

    dims = torch.arange(0, head_dim, 2, dtype=torch.float32, device=positions.device)
    inv_freq = 1.0 / (theta ** (dims / head_dim))
    angles = positions.to(torch.float32).unsqueeze(-1) * inv_freq  # [T, d/2]
    angles = torch.cat((angles, angles), dim=-1).to(torch.float64)
    return angles.cos().to(dtype), angles.sin().to(dtype)


def rotate(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x' = x*cos + rot(x)*sin with rot(x) = cat(-x[d/2:], x[:d/2]); pairs are
    (i, i + d/2) (mini_llm/nn/rope.py:110-114, 142-146).  x: [T, heads, d]."""

    half = x.shape[-1] // 2
    rotated = torch.cat((-x[..., half:], x[..., :half]), dim=-1)
    return x * cos.unsqueeze(1) + rotated * sin.unsqueeze(1)


def causal_attention(q, k, v, scale: float, window: int | None = None) -> torch.Tensor:
    """Per query head j, with KV head j // (nq/nkv): S = q k^T * scale, key t visible
    iff t <= query position, softmax over visible keys, o = P v
    (mini_llm/nn/attention.py:18-33, 95-99, 231-248).  q: [T, nq, d]; k, v: [T, nkv, d].
    ``window`` (not used by Qwen3) keeps only keys t > p - window."""

    T, nq, d = q.shape
    nkv = k.shape[1]
    group = nq // nkv
    out = torch.empty_like(q)
    idx = torch.arange(T, device=q.device)
    visible = idx.view(1, T) <= idx.view(T, 1)
    if window is not None:
        visible &= idx.view(1, T) > idx.view(T, 1) - window
    for head in range(nq):
        kv = head // group
        scores = (q[:, head] @ k[:, kv].T) * scale  # [T, T]
        scores = scores.masked_fill(~visible, float("-inf"))
        scores = scores - scores.max(dim=-1, keepdim=True).values
        weights = scores.exp()
        weights = weights / weights.sum(dim=-1, keepdim=True)
        out[:, head] = weights @ v[:, kv]
    return out


def attention_block(x, w: Mapping[str, torch.Tensor], prefix: str, cfg, cos, sin, store=_keep) -> torch.Tensor:
    """q/k/v projections, head split, per-head q/k RMSNorm before rotary, rotation,
    causal GQA attention, merge heads, output projection without bias
    (mini_llm/nn/attention.py:161-181, 250-254, 291-302)."""

    nq, nkv, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    T = x.shape[0]
    q = x @ w[f"{prefix}.q_proj.weight"].T
    k = x @ w[f"{prefix}.k_proj.weight"].T
    v = x @ w[f"{prefix}.v_proj.weight"].T
    if cfg.get("attention_bias", False):
        q = q + w[f"{prefix}.q_proj.bias"]
        k = k + w[f"{prefix}.k_proj.bias"]
        v = v + w[f"{prefix}.v_proj.bias"]
    q, k, v = store(q).view(T, nq, d), store(k).view(T, nkv, d), store(v).view(T, nkv, d)
    q = rms_norm(q, w[f"{prefix}.q_norm.weight"], cfg["rms_norm_eps"])
    k = rms_norm(k, w[f"{prefix}.k_norm.weight"], cfg["rms_norm_eps"])
    q, k = store(rotate(q, cos, sin)), store(rotate(k, cos, sin))
    o = store(causal_attention(q, k, v, 1.0 / math.sqrt(d)))
    return o.reshape(T, nq * d) @ w[f"{prefix}.o_proj.weight"].T


def swiglu(x, w: Mapping[str, torch.Tensor], prefix: str, store=_keep) -> torch.Tensor:
    """down(silu(gate(x)) * up(x)), silu(z) = z * sigmoid(z), no biases
    (mini_llm/nn/mlp.py:80-87)."""

    gate = x @ w[f"{prefix}.gate_proj.weight"].T
    up = x @ w[f"{prefix}.up_proj.weight"].T
    return store((gate / (1.0 + torch.exp(-gate))) * up) @ w[f"{prefix}.down_proj.weight"].T


def decoder_layer(h, w, layer: int, cfg, cos, sin, store=_keep) -> torch.Tensor:
    """Pre-norm block: h = h + Attn(norm_in(h)); h = h + MLP(norm_post(h))
    (mini_llm/model/qwen.py:58-72)."""

    p = f"model.layers.{layer}"
    eps = cfg["rms_norm_eps"]
    h = h + attention_block(store(rms_norm(h, w[f"{p}.input_layernorm.weight"], eps)), w, f"{p}.self_attn", cfg, cos, sin, store)
    h = h + swiglu(store(rms_norm(h, w[f"{p}.post_attention_layernorm.weight"], eps)), w, f"{p}.mlp", store)
    return h


def forward(weights: Mapping[str, torch.Tensor], cfg: Mapping, token_ids, dtype=torch.float32, *, rows=None,
            store=_keep) -> torch.Tensor:
    """Logits [T, vocab] (or only at the positions ``rows``) for one whole sequence starting at position 0: embedding
    without scaling, rotary tables once, the layers in order, the final norm on every
    row, the output head without bias (mini_llm/model/base.py:72-89,
    mini_llm/model/qwen.py:112).  A tied head (no ``lm_head.weight`` stored) uses the
    embedding matrix."""

    w = {name: t.to(dtype) for name, t in weights.items()}
    device = w["model.embed_tokens.weight"].device
    ids = torch.as_tensor(token_ids, dtype=torch.long, device=device)
    h = w["model.embed_tokens.weight"][ids]
    cos, sin = rotary_tables(torch.arange(ids.shape[0], device=device), cfg["head_dim"], float(cfg["rope_theta"]), dtype)
    for layer in range(cfg["num_hidden_layers"]):
        h = decoder_layer(h, w, layer, cfg, cos, sin, store)
    if rows is not None:
        h = h[torch.as_tensor(rows, dtype=torch.long, device=device)]
    h = store(rms_norm(h, w["model.norm.weight"], cfg["rms_norm_eps"]))
    head = w.get("lm_head.weight", w["model.embed_tokens.weight"])
    return h @ head.T
