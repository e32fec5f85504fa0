"""Plain next-token selection: the reference's filters (mini_llm/sampling.py:40-69)
with sorting, and the engine's documented noise (splitmix64-keyed uniforms turned
into Gumbel noise) written with Python integers.  Shares no code with the engine."""

from __future__ import annotations

import math

import torch

_M = (1 << 64) - 1


def splitmix64(z: int) -> int:
    z = (z + 0x9E3779B97F4A7C15) & _M
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _M
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _M
    return z ^ (z >> 31)


def uniforms(seed: int, counter: int, vocab: int) -> torch.Tensor:
    """u_i = (top 23 bits of splitmix64(stream + i * c) + 0.5) / 2^23,
    stream = splitmix64(seed ^ splitmix64(counter))."""

    stream = splitmix64(seed ^ splitmix64(counter))
    values = [((splitmix64((stream + i * 0xD1B54A32D192ED03) & _M) >> 41) + 0.5) / 8388608.0 for i in range(vocab)]
    return torch.tensor(values, dtype=torch.float64)


def kept_mask(logits: torch.Tensor, temperature: float, top_k: int | None, top_p: float) -> torch.Tensor:
    """Which tokens survive top-k then top-p (mini_llm/sampling.py:51-68): after
    dividing by the temperature, keep the k largest; sort descending, softmax,
    drop a token iff the cumulative probability *before* it is >= top_p."""

    x = logits.double() / temperature
    keep = torch.ones_like(x, dtype=torch.bool)
    if top_k is not None and top_k < x.numel():
        kth = torch.topk(x, top_k).values[-1]
        keep &= x >= kth
    if top_p < 1.0:
        masked = x.masked_fill(~keep, float("-inf"))
        order = torch.argsort(masked, descending=True)
        probs = torch.softmax(masked[order], dim=-1)
        before = torch.cumsum(probs, dim=-1) - probs
        drop = before >= top_p
        keep[order[drop]] = False
    return keep


def sample(logits: torch.Tensor, temperature: float, top_k: int | None, top_p: float, seed: int, counter: int):
    """Return (token, perturbed scores).  Greedy when temperature == 0."""

    if temperature == 0:
        return int(torch.argmax(logits)), logits.double()
    keep = kept_mask(logits, temperature, top_k, top_p)
    u = uniforms(seed, counter, logits.numel())
    scores = logits.double() / temperature - torch.log(-torch.log(u))
    scores = scores.masked_fill(~keep, float("-inf"))
    return int(torch.argmax(scores)), scores
