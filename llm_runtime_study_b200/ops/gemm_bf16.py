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
        "b200_gemm_tcgen05": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                              c_int, c_int, c_int, c_void_p, c_void_p, c_void_p],
        "b200_gemm_tcgen05_error": [],
        "b200_gemm_tcgen05_splitk_shape": [c_int, c_int, c_int, c_int, c_void_p, c_void_p],
        "b200_gemm_tcgen05_streamk_partial_floats": [],
        "b200_gemm_tcgen05_streamk_flags": [],
    },
)

native.register_library(
    "b200_gemm_skinny", ("gemm_skinny.cu",),
    {
        "b200_gemm_skinny": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p],
        "b200_gemm_skinny_variant": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                     c_void_p, c_void_p],
        "b200_gemm_skinny_residual": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p,
                                      native.c_float, c_void_p, c_void_p, c_void_p, c_void_p],
        "b200_gemm_skinny_partial_floats": [c_int],
    },
)

PAIR_MIN_ROWS = 256   # from here on pairs of SMs work on 256 x 256 tiles (tcgen05 cta_group::2)
PAIR_ENABLED = os.environ.get("LLM_RUNTIME_STUDY_B200_GEMM_PAIR", "1") != "0"
SKINNY_M = 16         # up to here weights are streamed straight into mma.sync fragments
KERNELS = {"persistent": 0, "pair": 1, "streamk": 2, "splitk": 3}

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


def supported(m: int, n: int, k: int) -> bool:
    """TMA needs rows that start on 16-byte boundaries: K a multiple of 8."""

    return k % 8 == 0 and m > 0 and n > 0


def pick_kernel(m: int, n: int, k: int) -> tuple[str, int]:
    """Which kernel and which tile width take a product of this shape (chosen from timings at the
    Qwen3-8B layer widths with 128 to 4,096 rows).  Pairs of SMs on 256 x 256 tiles when those fill
    most of the 74 pairs; one CTA per 128 x 256 tile when those cover half the SMs or more; up to
    256 rows and a third of the SMs: clusters that share a tile's K range (split-K, which chooses
    its own width); stream-K when a third of the SMs or fewer would have a tile and the K range is
    long enough to share; else one CTA per 128 x 128 tile.  A product with few tiles is as slow as
    the SM that has most to pull in, so it pays to spread the bytes over more SMs."""

    sms = native.sm_count()
    if m >= PAIR_MIN_ROWS and PAIR_ENABLED and 5 * -(-m // 256) * -(-n // 256) >= 2 * sms:   # 60 of a B200's 74 pairs
        return "pair", 256
    tiles = -(-m // 128) * -(-n // 256)
    if 2 * tiles >= sms:
        return "persistent", 256
    if m <= 256 and 3 * tiles <= sms:
        return "splitk", 0
    if 3 * tiles <= sms + 2 and k >= 48 * 64:
        return "streamk", 256
    return "persistent", 128


# weight elements from which 9 to 16 rows go to the tcgen05 split-K kernel
SKINNY_LARGE = int(os.environ.get("LLM_RUNTIME_STUDY_B200_SKINNY_LARGE", 52_000_000))


def splitk_shape(m: int, n: int, k: int, sm_count: int = 0) -> tuple[int, int]:
    """(tile width, CTAs per tile) the split-K kernel chooses by itself for this product."""

    import ctypes

    width, splits = ctypes.c_int(0), ctypes.c_int(0)
    native.call("b200_gemm_tcgen05_splitk_shape", m, n, k, sm_count or native.sm_count(), ctypes.addressof(width), ctypes.addressof(splits), launches=0)
    return width.value, splits.value


def few_rows_kernel(m: int, n: int, k: int) -> str:
    """"skinny" or "splitk" for at most ``SKINNY_M`` rows.  The weight-streaming kernel handles 9 to 16
    rows as two token tiles per weight fragment and then reaches about 5 TB/s; the split-K kernel
    streams at 6 TB/s but costs about 4 us more per launch, so it takes the products whose weights
    are larger than about 100 MB (Qwen3-32B at 16 rows: 178 against 205 us per layer; Qwen3-8B
    gate/up: 37 against 43 us), and the weight-streaming kernel the rest.  Up to 8 rows the
    weight-streaming kernel is as fast or faster except where few output rows meet a very long K
    (the down projections of Qwen3-14B and 32B: 33.6 against 36.9 us, 47.0 against 52.9 us)."""

    if m > 8:
        return "splitk" if n * k >= SKINNY_LARGE else "skinny"
    return "splitk" if k >= 16384 and n * k >= SKINNY_LARGE else "skinny"


def linear(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None,
           out_dtype: torch.dtype = torch.bfloat16, *, swiglu: bool = False, add_to: torch.Tensor | None = None,
           kernel: str | None = None, tile_n: int | None = None, splits: int = 0, stages: int = 0) -> torch.Tensor:
    """``x @ weight.T (+ bias)`` on the tcgen05 tensor cores; float32 accumulation; bfloat16 or
    float32 output.

    ``swiglu``: the weight holds gate and up rows interleaved in blocks of eight and the result is
    ``silu(gate) * up``, half as wide.  ``add_to`` (float32 ``[M, N]``): the product is added to it
    in place and it is returned.  ``kernel``: "persistent" (one CTA per tile of 128 rows and
    ``tile_n`` = 128 or 256 columns), "pair" (two CTAs per 256 x 256 tile), "streamk" (few
    tiles: up to three SMs share a tile's K range) or "splitk" (few rows: a cluster of ``splits``
    <= 8 CTAs shares the K range of every 128 x ``tile_n`` tile, ``tile_n`` a multiple of 32; 0 for either
    lets the kernel choose so that the SMs are filled once; ``stages``: depth of its operand ring, 0 = as
    deep as shared memory allows); chosen by shape when not given."""

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
    picked_kernel, picked_width = pick_kernel(m, n, k)
    kernel = kernel or picked_kernel
    if kernel == "splitk":
        tile_n = tile_n or 0                        # 0: the kernel chooses
        if tile_n % 32 or not 0 <= tile_n <= 256 or not 0 <= splits <= 8:
            raise KernelError(f"split-K takes tiles of 32 to 256 columns in steps of 32 and up to 8 CTAs per tile, got {tile_n}, {splits}")
    else:
        tile_n = tile_n or (picked_width if kernel == picked_kernel else 256)
        if kernel not in KERNELS or tile_n not in (128, 256) or (tile_n == 128 and kernel != "persistent"):
            raise KernelError(f"unknown projection kernel {kernel!r} or tile width {tile_n}: expected one of {sorted(KERNELS)}, "
                              "256 columns, or 128 with the persistent kernel")
    partials, flags = _streamk_workspace(x.device) if kernel == "streamk" else (None, None)
    native.call("b200_gemm_tcgen05", x.data_ptr(), weight.data_ptr(), native.ptr(bias), out.data_ptr(), m, n, k,
                out.shape[1], 1 if out_dtype == torch.float32 else 0, 1 if swiglu else 0, 0 if add_to is None else 1,
                KERNELS[kernel], tile_n, splits, stages, native.ptr(partials), native.ptr(flags), native.stream_ptr())
    return out


native.register_error_probe("b200_gemm_tcgen05", "b200_gemm_tcgen05_error", "tcgen05 projection")


def check_error() -> None:
    """Synchronise and raise if a bounded wait inside the kernel ran out."""

    code = native.query("b200_gemm_tcgen05_error")
    if code:
        where = {1: "producer", 2: "tensor-core issue", 3: "epilogue", 4: "accumulator buffer", 5: "flag of a shared tile",
                 -1: "device error"}.get(code, str(code))
        for _, flags in _STREAMK_WORKSPACE.values():     # a wait that ran out may have left flags behind
            flags.zero_()
        raise KernelError(f"tcgen05 projection: a bounded wait ran out ({where})")


def linear_skinny(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None,
                  out_dtype: torch.dtype = torch.bfloat16, *, variant: int = 0, swiglu: bool = False,
                  row_scale: torch.Tensor | None = None) -> torch.Tensor:
    """``x @ weight.T (+ bias)`` for at most 16 rows of ``x``: the weight-streaming kernel.
    ``swiglu``: see ``linear``.  ``row_scale`` (float32 ``[16]``): the rows of ``x`` still lack these factors
    (an RMS norm left half done, see ``linear_skinny_residual``); they are applied to the product, before the bias."""

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
    if row_scale is not None:
        native.require(row_scale, "row_scale", dtype=torch.float32, shape=(16,))
    width = n // 2 if swiglu else n
    out = torch.empty((m, width), dtype=out_dtype, device=x.device)
    native.call("b200_gemm_skinny_variant", x.data_ptr(), weight.data_ptr(), native.ptr(bias), out.data_ptr(), m, n, k, width,
                1 if out_dtype == torch.float32 else 0, variant, 1 if swiglu else 0, native.ptr(row_scale), native.stream_ptr())
    return out


def linear_skinny_residual(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None, resid: torch.Tensor,
                           next_weight: torch.Tensor, eps: float) -> tuple[torch.Tensor, torch.Tensor]:
    """``resid += x @ weight.T (+ bias)`` in place (float32 ``[M, N]``, at most 16 rows), and on the way out
    what the RMS norm after it needs: ``resid * next_weight`` rounded to bfloat16, and every row's factor
    ``rsqrt(mean of squares + eps)`` (``[16]`` floats; rows from ``M`` on hold 0).  Returns (weighted, row_scale)."""

    native.require(x, "x", dtype=torch.bfloat16, dims=2)
    native.require(weight, "weight", dtype=torch.bfloat16, dims=2)
    m, k = x.shape
    n = weight.shape[0]
    if weight.shape[1] != k or m > SKINNY_M or k % 8:
        raise KernelError(f"the weight-streaming kernel takes at most {SKINNY_M} rows and K a multiple of 8; got {m}, {k}")
    native.require(resid, "resid", dtype=torch.float32, shape=(m, n))
    native.require(next_weight, "next_weight", dtype=torch.float32, shape=(n,))
    if bias is not None:
        native.require(bias, "bias", dtype=torch.float32, shape=(n,))
    weighted = torch.empty((m, n), dtype=torch.bfloat16, device=x.device)
    row_scale = torch.empty(16, dtype=torch.float32, device=x.device)
    partials = torch.empty(native.query("b200_gemm_skinny_partial_floats", n), dtype=torch.float32, device=x.device)
    native.call("b200_gemm_skinny_residual", x.data_ptr(), weight.data_ptr(), native.ptr(bias), resid.data_ptr(), m, n, k, n,
                next_weight.data_ptr(), float(eps), weighted.data_ptr(), row_scale.data_ptr(), partials.data_ptr(),
                native.stream_ptr(), launches=2)
    return weighted, row_scale
