"""Sampling options, with the reference's names, defaults and checks
(mini_llm/sampling.py:15-37)."""

from __future__ import annotations

import math
from dataclasses import dataclass

from ..errors import SamplingError


@dataclass(frozen=True, slots=True)
class SamplingConfig:
    """``temperature = 0`` picks the largest logit.  A positive temperature draws
    from ``softmax(logits / temperature)``, optionally restricted to the ``top_k``
    largest logits and then to the smallest set of most probable tokens whose mass
    reaches ``top_p``.  ``seed`` makes a request's draws reproducible and
    independent of what else is in the batch; without it a fresh seed is drawn
    for every request."""

    temperature: float = 0.0
    top_k: int | None = None
    top_p: float = 1.0
    seed: int | None = None

    def __post_init__(self) -> None:
        if not math.isfinite(self.temperature) or self.temperature < 0:
            raise SamplingError("temperature must be finite and non-negative")
        if self.top_k is not None and self.top_k <= 0:
            raise SamplingError("top_k must be positive when supplied")
        if not math.isfinite(self.top_p) or not 0 < self.top_p <= 1:
            raise SamplingError("top_p must satisfy 0 < top_p <= 1")
        if self.seed is not None and self.seed < 0:
            raise SamplingError("seed must be non-negative when supplied")
