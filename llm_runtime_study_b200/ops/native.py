"""Loader of the native kernel libraries and thin typed wrappers over them.

Every wrapper checks shapes, dtypes, contiguity and device on the host, then
calls the C entry point with raw device pointers and the current CUDA stream.
There is no other implementation behind these functions: if the library cannot
be built or loaded, or a tensor is not on a CUDA device, a ``KernelError`` is
raised.
"""

from __future__ import annotations

import ctypes
import os
from typing import Sequence

import torch

from ..csrc.build import load_library
from ..errors import KernelError

c_int, c_float, c_void_p = ctypes.c_int, ctypes.c_float, ctypes.c_void_p

DTYPE_TAG = {torch.float32: 0, torch.bfloat16: 1}

_OWN_ERRORS = {
    10001: "a size argument is not supported by this kernel",
    10002: "unsupported storage type",
    10003: "a size exceeds what this kernel can hold on chip",
    10004: "scratch buffer too small",
}

# library name -> (sources, {function: argument types})
_LIBRARIES = {
    "b200_elementwise": (
        ("elementwise.cu",),
        {
            "b200_embedding": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_int, c_void_p],
            "b200_embedding_weighted": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float,
                                        c_float, c_int, c_void_p],
            "b200_add_rmsnorm": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_int, c_int, c_void_p],
            "b200_silu_mul": [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
            "b200_silu_mul_interleaved": [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
            "b200_qk_norm_rope_write": [
                c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_int, c_void_p, c_void_p,
                c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p,
            ],
        },
    ),
    "b200_gemm_f32": (
        ("gemm_f32.cu",),
        {"b200_gemm_f32": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p]},
    ),
    "b200_attention_simt": (
        ("attention_simt.cu",),
        {
            "b200_paged_attention_simt": [
                c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p,
            ],
        },
    ),
}

_functions: dict[str, ctypes._CFuncPtr] = {}


_DEFINES: dict[str, tuple[str, ...]] = {}
# Which small kernels release their successor at their first instruction (see pdl_launch_dependents
# in csrc/common.cuh): the norms (a projection follows and fetches weights meanwhile) and the rotary
# write (decode attention follows and asks for the pages of earlier steps meanwhile).
_early = os.environ.get("LLM_RUNTIME_STUDY_B200_EARLY", "norm,rope")
_DEFINES["b200_elementwise"] = tuple(f"B200_EARLY_{w.upper()}" for w in _early.split(",") if w and w != "none")


def library_specs() -> dict:
    """Sources of every library, for the build-everything entry point."""

    return {name: sources for name, (sources, _) in _LIBRARIES.items()}


def library_loaded(name: str) -> bool:
    """Whether any function of this library has been looked up (and the library therefore loaded)."""

    return any(key.startswith(name + ":") or (key in _LIBRARIES.get(name, ((), {}))[1]) for key in _functions)


def library_defines(name: str) -> tuple[str, ...]:
    return _DEFINES.get(name, ())


def _function(name: str, library: str | None = None):
    """The C function ``name``; ``library`` picks among libraries that export
    the same symbol (one build per head size)."""

    key = name if library is None else f"{library}:{name}"
    fn = _functions.get(key)
    if fn is None:
        for lib_name, (sources, table) in _LIBRARIES.items():
            if name in table and library in (None, lib_name):
                lib = load_library(lib_name, sources, _DEFINES.get(lib_name, ()))
                for fname, argtypes in table.items():
                    f = getattr(lib, fname)
                    f.argtypes = argtypes
                    f.restype = ctypes.c_long if fname.endswith("_floats") else c_int
                    _functions[fname if library is None else f"{lib_name}:{fname}"] = f
                break
        else:
            raise KernelError(f"no native library provides {name}")
        fn = _functions[key]
    return fn


def register_library(lib_name: str, sources: Sequence[str], table: dict, defines: Sequence[str] = ()) -> None:
    """Add a library (used by kernels that are built per head size)."""

    _LIBRARIES[lib_name] = (tuple(sources), dict(table))
    _DEFINES[lib_name] = tuple(defines)


def check(status: int, what: str) -> None:
    if status == 0:
        return
    if status in _OWN_ERRORS:
        raise KernelError(f"{what}: {_OWN_ERRORS[status]}")
    raise KernelError(f"{what}: CUDA error {status} (cudaError_t)")


_launches = 0


def launch_count() -> int:
    """How many of this package's kernels have been launched (graph replays
    count every kernel they hold)."""

    return _launches


def add_launches(n: int) -> None:
    global _launches
    _launches += n


def call(name: str, *args, library: str | None = None, launches: int = 1) -> None:
    global _launches
    _launches += launches
    check(_function(name, library)(*args), name)


def query(name: str, *args, library: str | None = None) -> int:
    """Call a C function that returns a number rather than a status."""

    return _function(name, library)(*args)


B200_SM_COUNT = 148
_sm_counts: dict[int, int] = {}


def sm_count() -> int:
    """Streaming multiprocessors of the current CUDA device (a B200's 148 where no device is visible,
    so that the host-side rules that choose kernels can be exercised without one)."""

    if not torch.cuda.is_available():
        return B200_SM_COUNT
    device = torch.cuda.current_device()
    count = _sm_counts.get(device)
    if count is None:
        count = _sm_counts[device] = torch.cuda.get_device_properties(device).multi_processor_count
    return count


# (library, C function returning a status word, what a non-zero word means)
_ERROR_PROBES: list[tuple[str, str, str]] = []


def register_error_probe(library: str, function: str, what: str) -> None:
    """A library whose kernels bound their waits keeps a status word on the device; ``function``
    (no arguments, synchronises) returns it."""

    if (library, function, what) not in _ERROR_PROBES:
        _ERROR_PROBES.append((library, function, what))


def check_kernel_errors() -> None:
    """Raise ``KernelError`` if a bounded wait inside any loaded kernel library ever ran out.  A kernel
    whose wait ran out finishes on incomplete data, so what it wrote must not be used."""

    for library, function, what in list(_ERROR_PROBES):
        if not library_loaded(library):
            continue
        code = query(function, library=library)
        if code:
            raise KernelError(f"{what}: a bounded wait ran out inside the kernel (status {code}); its results are invalid")


def stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


def ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def require(t: torch.Tensor, name: str, *, dtype=None, shape=None, dims=None) -> torch.Tensor:
    if not isinstance(t, torch.Tensor) or t.device.type != "cuda":
        raise KernelError(f"{name} must be a CUDA tensor: the kernels have no other path")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    if dtype is not None:
        allowed = dtype if isinstance(dtype, (tuple, list)) else (dtype,)
        if t.dtype not in allowed:
            raise KernelError(f"{name} has dtype {t.dtype}, expected {allowed}")
    if dims is not None and t.dim() != dims:
        raise KernelError(f"{name} has {t.dim()} dimensions, expected {dims}")
    if shape is not None and tuple(t.shape) != tuple(shape):
        raise KernelError(f"{name} has shape {tuple(t.shape)}, expected {tuple(shape)}")
    return t


def tag(dtype: torch.dtype) -> int:
    try:
        return DTYPE_TAG[dtype]
    except KeyError:
        raise KernelError(f"unsupported storage type {dtype}; expected float32 or bfloat16") from None
