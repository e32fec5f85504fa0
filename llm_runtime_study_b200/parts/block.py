"""Arrangement of norm, mixer and feed-forward in one layer."""

from __future__ import annotations

from typing import Any, Mapping

import torch

from ..weights.checkpoint import TensorSpec
from ..weights.view import TensorView
from .base import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, Block, ResidualStream, Runtime

_DEFAULT_NAMES = {
    "mixer_norm": "input_layernorm",
    "mixer": "self_attn",
    "ffn_norm": "post_attention_layernorm",
    "feed_forward": "mlp",
}


@BLOCKS.register("pre_norm")
class PreNormBlock(Block):
    """``h = h + mixer(norm_1(h)); h = h + ffn(norm_2(h))``
    (mini_llm/model/qwen.py:58-72).  The additions are carried out by the *next*
    norm, in float32, while it reads the rows anyway.  ``names`` gives the
    checkpoint's name of each sub-part below the layer's prefix."""

    def __init__(
        self, *, mixer: Mapping[str, Any], feed_forward: Mapping[str, Any], mixer_norm: Mapping[str, Any],
        ffn_norm: Mapping[str, Any], names: Mapping[str, str] | None = None,
    ) -> None:
        self.names = {**_DEFAULT_NAMES, **(names or {})}
        self.mixer = MIXERS.build(mixer)
        self.feed_forward = FEED_FORWARDS.build(feed_forward)
        self.mixer_norm = NORMS.build(mixer_norm)
        self.ffn_norm = NORMS.build(ffn_norm)

    graph_safe = True

    def children(self):
        return (self.mixer_norm, self.mixer, self.ffn_norm, self.feed_forward)

    def _parts(self):
        return (
            (self.names["mixer_norm"], self.mixer_norm),
            (self.names["mixer"], self.mixer),
            (self.names["ffn_norm"], self.ffn_norm),
            (self.names["feed_forward"], self.feed_forward),
        )

    def tensor_specs(self) -> dict[str, TensorSpec]:
        return {f"{prefix}.{n}": s for prefix, part in self._parts() for n, s in part.tensor_specs().items()}

    def load(self, tensors: Mapping[str, torch.Tensor], runtime: Runtime) -> None:
        self.runtime = runtime
        view = TensorView.of(tensors)
        for prefix, part in self._parts():
            part.load(view.sub(prefix), runtime)

    fuses_norms = True

    def first_norm(self):
        return self.mixer_norm

    def forward(self, stream: ResidualStream, ctx: Any, cache: Any, next_norm: Any = None) -> None:
        x = stream.take_rows(self.mixer_norm, self.mixer)
        stream.put(self._run(self.mixer, (x, ctx, cache), stream.resid, self.ffn_norm), self.ffn_norm)
        x = stream.take_rows(self.ffn_norm, self.feed_forward)
        stream.put(self._run(self.feed_forward, (x, ctx), stream.resid, next_norm), next_norm)

    @staticmethod
    def _run(part: Any, args: tuple, resid: torch.Tensor, next_norm: Any):
        """Call a mixer or feed-forward with as much as it says it can take."""

        if not part.adds_to_residual:
            return part.forward(*args)
        if part.fuses_norms:
            return part.forward(*args, residual=resid, next_norm=next_norm)
        return part.forward(*args, residual=resid)
