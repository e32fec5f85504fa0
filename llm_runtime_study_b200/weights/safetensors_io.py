"""Reading and writing safetensors files without a library.

A safetensors file is an 8-byte little-endian header length, a JSON header that
maps tensor names to ``{"dtype", "shape", "data_offsets"}``, and the raw tensor
bytes.  The reference inspects headers first and leaves payloads unmapped until
a tensor is asked for (mini_llm/checkpoint.py:62-68, :139-164); so does this
module: ``read_header`` touches only the header, ``map_tensor`` maps the bytes of one
tensor, and ``read_tensors`` returns copies that outlive the files.
"""

from __future__ import annotations

import json
import mmap
import struct
from dataclasses import dataclass
from pathlib import Path
from typing import Iterable, Mapping

import torch

from ..errors import CheckpointError

# safetensors dtype string -> (torch dtype, bytes per element)
_DTYPES: dict[str, tuple[torch.dtype, int]] = {
    "F64": (torch.float64, 8),
    "F32": (torch.float32, 4),
    "F16": (torch.float16, 2),
    "BF16": (torch.bfloat16, 2),
    "I64": (torch.int64, 8),
    "I32": (torch.int32, 4),
    "I16": (torch.int16, 2),
    "I8": (torch.int8, 1),
    "U8": (torch.uint8, 1),
    "BOOL": (torch.bool, 1),
}
_TO_NAME = {dtype: name for name, (dtype, _) in _DTYPES.items()}

FLOAT_DTYPES = ("F64", "F32", "F16", "BF16")
INT_DTYPES = ("I64", "I32", "I16", "I8", "U8")


@dataclass(frozen=True, slots=True)
class TensorInfo:
    """Header entry of one stored tensor."""

    name: str
    shape: tuple[int, ...]
    dtype: str
    num_elements: int
    num_bytes: int
    path: Path
    begin: int  # byte offset of the payload inside the file


def read_header(path: str | Path) -> list[TensorInfo]:
    """Return the header entries of one file, sorted by tensor name."""

    path = Path(path)
    if not path.is_file():
        raise CheckpointError(f"checkpoint file does not exist: {path}")
    if path.suffix != ".safetensors":
        raise CheckpointError(f"checkpoint must use the .safetensors extension: {path}")
    size = path.stat().st_size
    with open(path, "rb") as handle:
        prefix = handle.read(8)
        if len(prefix) != 8:
            raise CheckpointError(f"not a safetensors file (too short): {path}")
        (header_len,) = struct.unpack("<Q", prefix)
        if header_len <= 0 or 8 + header_len > size:
            raise CheckpointError(f"not a safetensors file (bad header length): {path}")
        try:
            header = json.loads(handle.read(header_len).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as exc:
            raise CheckpointError(f"not a safetensors file (bad header): {path}: {exc}") from exc
    if not isinstance(header, dict):
        raise CheckpointError(f"not a safetensors file (header is not an object): {path}")
    data_start = 8 + header_len
    infos = []
    for name, entry in header.items():
        if name == "__metadata__":
            continue
        try:
            dtype = entry["dtype"]
            shape = tuple(int(v) for v in entry["shape"])
            begin, end = (int(v) for v in entry["data_offsets"])
        except (KeyError, TypeError, ValueError) as exc:
            raise CheckpointError(f"bad header entry for {name!r} in {path}") from exc
        if dtype not in _DTYPES:
            raise CheckpointError(f"unsupported safetensors dtype {dtype!r} for {name!r} in {path}")
        count = 1
        for extent in shape:
            count *= extent
        num_bytes = count * _DTYPES[dtype][1]
        if end - begin != num_bytes or begin < 0 or data_start + end > size:
            raise CheckpointError(f"payload of {name!r} does not match its header in {path}")
        infos.append(TensorInfo(name, shape, dtype, count, num_bytes, path, data_start + begin))
    infos.sort(key=lambda info: info.name)
    return infos


def map_tensor(info: TensorInfo) -> torch.Tensor:
    """One stored tensor as a CPU tensor over a private mapping of just its bytes
    (nothing is copied; pages come in as they are read).  The mapping lives as long
    as the tensor does, so a loader that places one tensor after the other on the
    device never holds more of the file in memory than the tensors it still uses."""

    dtype = _DTYPES[info.dtype][0]
    if info.num_elements == 0:
        return torch.empty(info.shape, dtype=dtype)
    start = info.begin - info.begin % mmap.ALLOCATIONGRANULARITY
    with open(info.path, "rb") as handle:
        # a private (copy-on-write) mapping is writable as far as torch is concerned, and never written
        mapped = mmap.mmap(handle.fileno(), info.begin - start + info.num_bytes, access=mmap.ACCESS_COPY, offset=start)
    flat = torch.frombuffer(mapped, dtype=dtype, count=info.num_elements, offset=info.begin - start)
    return flat.reshape(info.shape)


def read_tensors(infos: Iterable[TensorInfo]) -> dict[str, torch.Tensor]:
    """Materialise tensors (CPU, stored dtype) as copies of their own, which stay
    valid when the files change or disappear."""

    return {info.name: map_tensor(info).clone() for info in infos}


def write_file(path: str | Path, tensors: Mapping[str, torch.Tensor]) -> None:
    """Write one safetensors file; tensors are laid out in sorted-name order,
    each payload starting on an 8-byte boundary of the data section."""

    path = Path(path)
    header: dict[str, dict] = {}
    offset = 0
    order = sorted(tensors)
    for name in order:
        tensor = tensors[name]
        if tensor.dtype not in _TO_NAME:
            raise CheckpointError(f"cannot store dtype {tensor.dtype} for {name!r}")
        num_bytes = tensor.numel() * tensor.element_size()
        header[name] = {
            "dtype": _TO_NAME[tensor.dtype],
            "shape": list(tensor.shape),
            "data_offsets": [offset, offset + num_bytes],
        }
        offset += num_bytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    with open(path, "wb") as handle:
        handle.write(struct.pack("<Q", len(blob)))
        handle.write(blob)
        for name in order:
            tensor = tensors[name].detach().contiguous().cpu()
            handle.write(tensor.view(torch.uint8).reshape(-1).numpy().tobytes()
                         if tensor.numel() else b"")
