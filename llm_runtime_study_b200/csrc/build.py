"""In-tree build of the CUDA sources into shared libraries for sm_100a.

Each library is one ``nvcc -shared`` call over plain ``extern "C"`` entry points
(no Python or torch headers, so a file compiles in seconds) and is loaded with
``ctypes``.  The object name carries a hash of the sources and flags, so an
edited kernel is never served by a stale binary.  Libraries live beside the
sources under ``csrc/_build/``; when that folder cannot be written (a read-only
install) a per-user folder under the system temporary directory is used.
While nvcc runs, a line is printed to stderr every few seconds.
"""

from __future__ import annotations

import ctypes
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path
from typing import Iterable, Sequence

from ..errors import KernelError

CSRC_DIR = Path(__file__).resolve().parent
ARCH_FLAGS = ("-gencode", "arch=compute_100a,code=sm_100a")
BASE_FLAGS = (
    "-O3", "-std=c++17", "-lineinfo", "-shared", "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr", "-Xptxas", "-v",
)

_loaded: dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()


def _nvcc() -> str:
    for candidate in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if candidate and Path(candidate).is_file():
            return candidate
    raise KernelError("nvcc was not found; the CUDA kernels cannot be built")


def _build_dir() -> Path:
    preferred = CSRC_DIR / "_build"
    try:
        preferred.mkdir(exist_ok=True)
        probe = preferred / f".probe-{os.getpid()}"
        probe.write_bytes(b"")
        probe.unlink()
        return preferred
    except OSError:
        fallback = Path(tempfile.gettempdir()) / f"llm_runtime_study_b200-build-{os.getuid()}"
        fallback.mkdir(parents=True, exist_ok=True)
        return fallback


def _digest(sources: Sequence[Path], flags: Sequence[str]) -> str:
    h = hashlib.sha256()
    for path in list(sources) + sorted(CSRC_DIR.glob("*.cuh")) + sorted(CSRC_DIR.glob("*.h")):
        h.update(path.name.encode())
        h.update(path.read_bytes())
    h.update(" ".join(flags).encode())
    return h.hexdigest()[:16]


def library_path(name: str, sources: Iterable[str], defines: Sequence[str] = ()) -> tuple[Path, list[str], list[Path]]:
    paths = [CSRC_DIR / s for s in sources]
    flags = [*ARCH_FLAGS, *BASE_FLAGS, *[f"-D{d}" for d in defines]]
    out = _build_dir() / f"lib{name}-{_digest(paths, flags)}.so"
    return out, flags, paths


def build_library(name: str, sources: Iterable[str], defines: Sequence[str] = (), *, verbose: bool = True) -> Path:
    """Compile (if not already built) and return the path of the library."""

    out, flags, paths = library_path(name, sources, defines)
    if out.is_file():
        return out
    tmp = out.with_suffix(f".tmp{os.getpid()}.so")
    command = [_nvcc(), *flags, "-o", str(tmp), *[str(p) for p in paths]]
    if verbose:
        print(f"[llm_runtime_study_b200] compiling {name} for sm_100a ...", file=sys.stderr, flush=True)
    started = time.time()
    process = subprocess.Popen(command, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    done = threading.Event()

    def _ticker() -> None:
        while not done.wait(10.0):
            if verbose:
                print(
                    f"[llm_runtime_study_b200] still compiling {name} ({time.time() - started:.0f} s)",
                    file=sys.stderr, flush=True,
                )

    ticker = threading.Thread(target=_ticker, daemon=True)
    ticker.start()
    try:
        log, _ = process.communicate()
    finally:
        done.set()
    if process.returncode != 0:
        tmp.unlink(missing_ok=True)
        raise KernelError(f"nvcc failed for {name}:\n{log}")
    (out.with_suffix(".log")).write_text(log)
    os.replace(tmp, out)
    for stale in out.parent.glob(f"lib{name}-*"):      # builds of earlier versions of the sources
        if stale.stem != out.stem:
            stale.unlink(missing_ok=True)
    if verbose:
        print(f"[llm_runtime_study_b200] built {out.name} in {time.time() - started:.1f} s", file=sys.stderr, flush=True)
    return out


def load_library(name: str, sources: Iterable[str], defines: Sequence[str] = ()) -> ctypes.CDLL:
    """Build on first use, then ``dlopen``.  Raises ``KernelError`` loudly when
    the library can be neither found nor built: there is no other code path."""

    sources = tuple(sources)
    key = name + "|" + ",".join(sources) + "|" + ",".join(defines)
    with _lock:
        lib = _loaded.get(key)
        if lib is None:
            path = build_library(name, sources, defines)
            try:
                lib = ctypes.CDLL(str(path))
            except OSError as exc:
                raise KernelError(f"cannot load {path}: {exc}") from exc
            _loaded[key] = lib
        return lib
