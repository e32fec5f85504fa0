"""bfloat16 projections on the 5th-generation tensor cores (tcgen05, TMEM, TMA)."""

from __future__ import annotations

import os

import torch

from ..errors import KernelError
from . import native
from .native import c_int, c_void_p

native.register_library(
    "b200_gemm_tcgen05", ("gemm_tcgen05.cu",),
    {
        "b200_gemm_tcgen05": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p],
        "b200_gemm_tcgen05_swiglu": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p],
        "b200_gemm_tcgen05_error": [],
        "b200_gemm_tcgen05_add": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
        "b200_gemm_tcgen05_pair": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p],
        "b200_gemm_tcgen05_streamk_partial_floats": [],
        "b200_gemm_tcgen05_streamk_flags": [],
        "b200_gemm_tcgen05_streamk": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                      c_void_p, c_void_p, c_void_p],
    },
)

native.register_library(
    "b200_gemm_skinny", ("gemm_skinny.cu",),
    {
        "b200_gemm_skinny": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p],
        "b200_gemm_skinny_variant": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p],
    },
)

PAIR_MIN_ROWS = 256   # from here on pairs of SMs work on 256 x 256 tiles (tcgen05 cta_group::2)
PAIR_ENABLED = os.environ.get("LLM_RUNTIME_STUDY_B200_GEMM_PAIR", "1") != "0"
SKINNY_M = 16         # up to here weights are streamed straight into mma.sync fragments
SMALL_M = 64          # up to here the weight is the row operand ("swapped")
_SM_COUNT = 148


_STREAMK_WORKSPACE: dict[tuple, tuple[torch.Tensor, torch.Tensor]] = {}


def _streamk_workspace(device: torch.device) -> tuple[torch.Tensor, torch.Tensor]:
    """Partial accumulators and flags of the stream-K kernel, one set per device, made on first
    use and kept.  The flags are zero between launches; launches on one device share the set and
    therefore must follow each other on one stream, which is how the engine runs."""

    key = (device.type, device.index)
    have = _STREAMK_WORKSPACE.get(key)
    if have is None:
        floats = native.query("b200_gemm_tcgen05_streamk_partial_floats")
        flags = native.query("b200_gemm_tcgen05_streamk_flags")
        have = (torch.empty(floats, dtype=torch.float32, device=device), torch.zeros(flags, dtype=torch.int32, device=device))
        _STREAMK_WORKSPACE[key] = have
    return have


def linear_streamk(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None,
                   out_dtype: torch.dtype = torch.bfloat16, *, swiglu: bool = False,
                   add_to: torch.Tensor | None = None) -> torch.Tensor:
    """``x @ weight.T (+ bias)`` with the (tile, K block) pairs spread evenly over the SMs.
    ``swiglu``: as in :func:`linear`.  ``add_to`` (float32 ``[M, N]``): the product is added to it
    in place and it is returned."""

    native.require(x, "x", dtype=torch.bfloat16, dims=2)
    native.require(weight, "weight", dtype=torch.bfloat16, dims=2)
    m, k = x.shape
    n = weight.shape[0]
    if weight.shape[1] != k:
        raise KernelError(f"linear: x has width {k}, weight expects {weight.shape[1]}")
    if not supported(m, n, k):
        raise KernelError(f"tcgen05 projection needs K to be a multiple of 8, got {k}")
    if bias is not None:
        native.require(bias, "bias", dtype=torch.float32, shape=(n,))
    if swiglu and n % 16:
        raise KernelError("the SwiGLU epilogue needs an even number of 8-feature blocks")
    if add_to is not None:
        if swiglu:
            raise KernelError("add_to and swiglu exclude each other")
        native.require(add_to, "add_to", dtype=torch.float32, shape=(m, n))
        out, out_dtype = add_to, torch.float32
    else:
        if out_dtype not in (torch.bfloat16, torch.float32):
            raise KernelError(f"unsupported output type {out_dtype}")
        out = torch.empty((m, n // 2 if swiglu else n), dtype=out_dtype, device=x.device)
    partials, flags = _streamk_workspace(x.device)
    native.call("b200_gemm_tcgen05_streamk", x.data_ptr(), weight.data_ptr(), native.ptr(bias), out.data_ptr(), m, n, k,
                out.shape[1], 1 if out_dtype == torch.float32 else 0, 1 if swiglu else 0, 0 if add_to is None else 1,
                partials.data_ptr(), flags.data_ptr(), native.stream_ptr())
    return out


def supported(m: int, n: int, k: int) -> bool:
    """TMA needs rows that start on 16-byte boundaries: K a multiple of 8."""

    return k % 8 == 0 and m > 0 and n > 0


def pick_splits(m: int, n: int, k: int) -> int:
    """Parts the K range is cut into (a cluster of that many CTAs) so that a
    small-M product still puts a CTA on every SM.  0: the large-M kernel."""

    if m > SMALL_M:
        return 0
    tiles = -(-n // 128)
    k_blocks = -(-k // 64)
    splits = max(1, min(8, _SM_COUNT // tiles, k_blocks // 8))
    return splits


def linear_pair(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None,
                out_dtype: torch.dtype = torch.bfloat16, *, swiglu: bool = False,
                add_to: torch.Tensor | None = None) -> torch.Tensor:
    """``x @ weight.T (+ bias)`` on pairs of SMs (tcgen05 ``cta_group::2``, 256 x 256 tiles).
    ``swiglu`` and ``add_to`` as in :func:`linear`."""

    native.require(x, "x", dtype=torch.bfloat16, dims=2)
    native.require(weight, "weight", dtype=torch.bfloat16, dims=2)
    m, k = x.shape
    n = weight.shape[0]
    if weight.shape[1] != k:
        raise KernelError(f"linear: x has width {k}, weight expects {weight.shape[1]}")
    if not supported(m, n, k):
        raise KernelError(f"tcgen05 projection needs K to be a multiple of 8, got {k}")
    if bias is not None:
        native.require(bias, "bias", dtype=torch.float32, shape=(n,))
    if swiglu and (n % 16 or add_to is not None):
        raise KernelError("the SwiGLU epilogue needs an even number of 8-feature blocks and excludes add_to")
    if add_to is not None:
        native.require(add_to, "add_to", dtype=torch.float32, shape=(m, n))
        out, out_dtype = add_to, torch.float32
    else:
        if out_dtype not in (torch.bfloat16, torch.float32):
            raise KernelError(f"unsupported output type {out_dtype}")
        out = torch.empty((m, n // 2 if swiglu else n), dtype=out_dtype, device=x.device)
    native.call("b200_gemm_tcgen05_pair", x.data_ptr(), weight.data_ptr(), native.ptr(bias), out.data_ptr(), m, n, k,
                out.shape[1], 1 if out_dtype == torch.float32 else 0, 1 if swiglu else 0, 0 if add_to is None else 1,
                native.stream_ptr())
    return out


def few_tiles(m: int, n: int, k: int) -> bool:
    """Products whose 128 x 256 tiles would occupy a third of the SMs or fewer, with a K range
    long enough to share: the stream-K kernel lets up to three SMs work on one tile."""

    tiles = -(-m // 128) * -(-n // 256)
    return 3 * tiles <= _SM_COUNT + 2 and k >= 48 * 64


def linear(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None,
           out_dtype: torch.dtype = torch.bfloat16, *, splits: int | None = None, swiglu: bool = False,
           add_to: torch.Tensor | None = None) -> torch.Tensor:
    """``x @ weight.T (+ bias)``; float32 accumulation; bfloat16 or float32 output.
    With ``swiglu`` the weight holds gate and up rows interleaved in blocks of eight and
    the result is ``silu(gate) * up``, half as wide (persistent kernel only).
    ``add_to`` (float32 ``[M, N]``): the product is added to it in place and it is returned."""

    if splits is None and x.dim() == 2 and weight.dim() == 2 and x.shape[0] > SMALL_M:
        if few_tiles(x.shape[0], weight.shape[0], x.shape[1]):
            return linear_streamk(x, weight, bias, out_dtype, swiglu=swiglu, add_to=add_to)
        if x.shape[0] >= PAIR_MIN_ROWS and PAIR_ENABLED:
            return linear_pair(x, weight, bias, out_dtype, swiglu=swiglu, add_to=add_to)

    native.require(x, "x", dtype=torch.bfloat16, dims=2)
    native.require(weight, "weight", dtype=torch.bfloat16, dims=2)
    m, k = x.shape
    n = weight.shape[0]
    if weight.shape[1] != k:
        raise KernelError(f"linear: x has width {k}, weight expects {weight.shape[1]}")
    if not supported(m, n, k):
        raise KernelError(f"tcgen05 projection needs K to be a multiple of 8, got {k}")
    if out_dtype not in (torch.bfloat16, torch.float32):
        raise KernelError(f"unsupported output type {out_dtype}")
    if bias is not None:
        native.require(bias, "bias", dtype=torch.float32, shape=(n,))
    if swiglu:
        if n % 16 or add_to is not None:
            raise KernelError("the SwiGLU epilogue needs an even number of 8-feature blocks and excludes add_to")
        out = torch.empty((m, n // 2), dtype=out_dtype, device=x.device)
        native.call("b200_gemm_tcgen05_swiglu", x.data_ptr(), weight.data_ptr(), native.ptr(bias), out.data_ptr(), m, n, k,
                    n // 2, 1 if out_dtype == torch.float32 else 0, native.stream_ptr())
        return out
    if add_to is not None:
        native.require(add_to, "add_to", dtype=torch.float32, shape=(m, n))
        native.call("b200_gemm_tcgen05_add", x.data_ptr(), weight.data_ptr(), native.ptr(bias), add_to.data_ptr(), m, n, k, n,
                    native.stream_ptr())
        return add_to
    out = torch.empty((m, n), dtype=out_dtype, device=x.device)
    if splits is None:
        splits = pick_splits(m, n, k)
    native.call("b200_gemm_tcgen05", x.data_ptr(), weight.data_ptr(), native.ptr(bias), out.data_ptr(), m, n, k, n,
                1 if out_dtype == torch.float32 else 0, splits, native.stream_ptr())
    return out


def check_error() -> None:
    """Synchronise and raise if a bounded wait inside the kernel ran out."""

    code = native.query("b200_gemm_tcgen05_error")
    if code:
        where = {1: "producer", 2: "tensor-core issue", 3: "epilogue", -1: "device error"}.get(code, str(code))
        raise KernelError(f"tcgen05 projection: a bounded wait ran out ({where})")


def linear_skinny(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None,
                  out_dtype: torch.dtype = torch.bfloat16, *, variant: int = 0, swiglu: bool = False) -> torch.Tensor:
    """``x @ weight.T (+ bias)`` for at most 16 rows of ``x``: the weight-streaming kernel.
    ``swiglu``: see ``linear``."""

    native.require(x, "x", dtype=torch.bfloat16, dims=2)
    native.require(weight, "weight", dtype=torch.bfloat16, dims=2)
    m, k = x.shape
    n = weight.shape[0]
    if weight.shape[1] != k:
        raise KernelError(f"linear: x has width {k}, weight expects {weight.shape[1]}")
    if m > SKINNY_M or k % 8:
        raise KernelError(f"the weight-streaming kernel takes at most {SKINNY_M} rows and K a multiple of 8; got {m}, {k}")
    if bias is not None:
        native.require(bias, "bias", dtype=torch.float32, shape=(n,))
    if swiglu and n % 16:
        raise KernelError("the SwiGLU epilogue needs an even number of 8-feature blocks")
    width = n // 2 if swiglu else n
    out = torch.empty((m, width), dtype=out_dtype, device=x.device)
    native.call("b200_gemm_skinny_variant", x.data_ptr(), weight.data_ptr(), native.ptr(bias), out.data_ptr(), m, n, k, width,
                1 if out_dtype == torch.float32 else 0, variant, 1 if swiglu else 0, native.stream_ptr())
    return out
