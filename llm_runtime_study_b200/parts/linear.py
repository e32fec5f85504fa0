"""Dense projections ``y = x W^T (+ b)`` with ``W`` stored ``[out, in]``."""

from __future__ import annotations

import os
from typing import Any

import torch

from ..errors import KernelError
from ..ops import functional as F
from ..ops import gemm_bf16
from .base import Runtime, WeightedRows


class Projection:
    """One weight matrix (possibly several checkpoint tensors stacked along the
    output axis, so that q/k/v or gate/up are one product) and an optional bias.

    float32 runtime: our FFMA kernel.  bfloat16 runtime, float32 accumulation,
    bfloat16 or float32 output:
      * up to 16 rows (decoding): our weight-streaming mma.sync kernel, or, for 9 to 16 rows
        and weights of more than about 100 MB, our tcgen05 split-K kernel
        (``gemm_bf16.few_rows_kernel``);
      * 128 rows and more (prompts): our tcgen05/TMEM/TMA kernels;
      * in between, and everywhere when ``LLM_RUNTIME_STUDY_B200_GEMM=library``: a
        library product (the reference's projections are ``nn.Linear``, i.e. library
        products: mini_llm/nn/attention.py:102-111), which is the faster one there;
        ``LLM_RUNTIME_STUDY_B200_GEMM_MID=splitk`` sends these row counts to our cluster
        split-K kernel instead.
    K must be a multiple of 8 for our bfloat16 kernels (16-byte rows); other
    widths go to the library product.

    The weight-streaming kernel also carries the RMS norms of a decode step: given
    ``add_to`` and ``next_norm`` it adds its product into the residual rows and returns
    ``WeightedRows`` prepared for that norm, and it takes ``WeightedRows`` as input,
    applying the norm's factor to its results (``FUSE_NORMS``, on by default;
    ``LLM_RUNTIME_STUDY_B200_FUSE_NORMS=0`` turns it off).
    """

    GEMM_BACKEND = os.environ.get("LLM_RUNTIME_STUDY_B200_GEMM", "tcgen05")
    TCGEN05_MIN_ROWS = 128
    MID_ROWS = os.environ.get("LLM_RUNTIME_STUDY_B200_GEMM_MID", "library")     # 17 to 127 rows: "library" or "splitk"
    FUSE_RESIDUAL = os.environ.get("LLM_RUNTIME_STUDY_B200_FUSE_RESIDUAL", "1") != "0"
    FUSE_NORMS = os.environ.get("LLM_RUNTIME_STUDY_B200_FUSE_NORMS", "1") != "0"

    def __init__(self, weights: list[torch.Tensor], biases: list[torch.Tensor] | None, runtime: Runtime) -> None:
        self.runtime = runtime
        # each tensor goes to the device as it is (possibly straight from a mapped file); stacking happens there
        placed = [runtime.place_matrix(w) for w in weights]
        self.weight = placed[0] if len(placed) == 1 else torch.cat(placed, dim=0)
        del placed
        self.out_features, self.in_features = self.weight.shape
        self.bias = None
        if biases:
            placed = [runtime.place_vector_f32(b) for b in biases]
            self.bias = placed[0] if len(placed) == 1 else torch.cat(placed, dim=0)

    def _streams(self, m: int) -> bool:
        """Whether ``m`` rows go to the weight-streaming kernel."""

        return (self.runtime.dtype == torch.bfloat16 and self.in_features % 8 == 0 and m <= gemm_bf16.SKINNY_M
                and not (self.GEMM_BACKEND == "tcgen05"
                         and gemm_bf16.few_rows_kernel(m, self.out_features, self.in_features) == "splitk"))

    def _unweighted(self, x: "torch.Tensor | WeightedRows") -> tuple[torch.Tensor, dict]:
        """Split an input into the rows to multiply and what the weight-streaming kernel needs to
        finish their norm; rows that go to another kernel are normalised here."""

        if not isinstance(x, WeightedRows):
            return x, {}
        if self._streams(x.values.shape[0]) and x.values.is_contiguous():
            return x.values, {"row_scale": x.scale}
        return x.normalised(), {}

    def swiglu(self, x: "torch.Tensor | WeightedRows") -> torch.Tensor:
        """For a projection whose rows are gate and up features interleaved in blocks of
        eight: ``silu(gate(x)) * up(x)`` in the activation type.  Our bfloat16 kernels apply
        the activation in their epilogue, so the ``[tokens, 2 I]`` intermediate is never
        written; the other paths run the projection and then the interleaved SiLU kernel."""

        x, norm = self._unweighted(x)
        if norm:
            return gemm_bf16.linear_skinny(x, self.weight, self.bias, torch.bfloat16, swiglu=True, **norm)
        if self.runtime.dtype == torch.bfloat16 and self.in_features % 8 == 0 and x.is_contiguous():
            m = x.shape[0]
            if m <= gemm_bf16.SKINNY_M:
                if self.GEMM_BACKEND == "tcgen05" and gemm_bf16.few_rows_kernel(m, self.out_features, self.in_features) == "splitk":
                    return gemm_bf16.linear(x, self.weight, self.bias, torch.bfloat16, swiglu=True, kernel="splitk")
                return gemm_bf16.linear_skinny(x, self.weight, self.bias, torch.bfloat16, swiglu=True)
            if self.GEMM_BACKEND == "tcgen05" and m >= self.TCGEN05_MIN_ROWS:
                return gemm_bf16.linear(x, self.weight, self.bias, torch.bfloat16, swiglu=True)
            if self.GEMM_BACKEND == "tcgen05" and self.MID_ROWS == "splitk":
                return gemm_bf16.linear(x, self.weight, self.bias, torch.bfloat16, swiglu=True, kernel="splitk")
        return F.silu_mul_interleaved(self(x))

    def __call__(self, x: "torch.Tensor | WeightedRows", out_dtype: torch.dtype | None = None, *,
                 add_to: torch.Tensor | None = None, next_norm: Any = None) -> "torch.Tensor | WeightedRows | None":
        """The projection of ``x``.  ``add_to`` (the float32 residual rows): where the kernel that takes
        this shape can add its result to them in its epilogue it does so and ``None`` is returned;
        otherwise the result is returned as always and the caller adds it.  ``next_norm`` (with
        ``add_to``): the norm that reads the residual rows next; where the kernel can, the rows are
        prepared for it on the way out and returned as ``WeightedRows`` (the product has been added)."""

        out_dtype = out_dtype or self.runtime.dtype
        x, norm = self._unweighted(x)
        if norm:
            return gemm_bf16.linear_skinny(x, self.weight, self.bias, out_dtype, **norm)
        if x.shape[-1] != self.in_features:
            raise KernelError(f"projection expects width {self.in_features}, got {x.shape[-1]}")
        if self.runtime.dtype == torch.float32:
            if out_dtype != torch.float32:
                raise KernelError("the float32 path keeps every activation in float32")
            return F.linear_f32(x, self.weight, self.bias)
        if x.dtype != torch.bfloat16:
            raise KernelError(f"bfloat16 projection got {x.dtype} input")
        m = x.shape[0]
        if self.in_features % 8 == 0 and x.is_contiguous():
            fusable = next_norm.fusable() if (next_norm is not None and self.FUSE_NORMS) else None
            if (fusable is not None and add_to is not None and out_dtype == torch.float32 and self._streams(m)
                    and fusable[0].shape[0] == self.out_features):
                return WeightedRows(*gemm_bf16.linear_skinny_residual(x, self.weight, self.bias, add_to, *fusable))
            if m <= gemm_bf16.SKINNY_M:
                if self.GEMM_BACKEND == "tcgen05" and gemm_bf16.few_rows_kernel(m, self.out_features, self.in_features) == "splitk":
                    if add_to is not None and out_dtype == torch.float32 and self.FUSE_RESIDUAL:
                        gemm_bf16.linear(x, self.weight, self.bias, torch.float32, add_to=add_to, kernel="splitk")
                        return None
                    return gemm_bf16.linear(x, self.weight, self.bias, out_dtype, kernel="splitk")
                return gemm_bf16.linear_skinny(x, self.weight, self.bias, out_dtype)
            if self.GEMM_BACKEND == "tcgen05" and m >= self.TCGEN05_MIN_ROWS:
                if add_to is not None and out_dtype == torch.float32 and self.FUSE_RESIDUAL:
                    gemm_bf16.linear(x, self.weight, self.bias, torch.float32, add_to=add_to)
                    return None
                return gemm_bf16.linear(x, self.weight, self.bias, out_dtype)
            if self.GEMM_BACKEND == "tcgen05" and self.MID_ROWS == "splitk":
                if add_to is not None and out_dtype == torch.float32 and self.FUSE_RESIDUAL:
                    gemm_bf16.linear(x, self.weight, self.bias, torch.float32, add_to=add_to, kernel="splitk")
                    return None
                return gemm_bf16.linear(x, self.weight, self.bias, out_dtype, kernel="splitk")
        if out_dtype == torch.bfloat16:
            y = torch.mm(x, self.weight.t())
        else:
            y = torch.mm(x, self.weight.t(), out_dtype=torch.float32)
        if self.bias is not None:
            y += self.bias.to(y.dtype)
        return y
