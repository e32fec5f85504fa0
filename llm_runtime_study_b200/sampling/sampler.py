"""Device-side sampling of one token per row of logits."""

from __future__ import annotations

import random
import struct
from typing import Sequence

import numpy as np
import torch

from ..errors import SamplingError
from ..ops import native
from .config import SamplingConfig

native.register_library(
    "b200_sampling", ("sampling.cu",),
    {
        "b200_sample": [native.c_void_p, native.c_int, native.c_int, native.c_void_p, native.c_void_p,
                        native.c_int, native.c_void_p],
        "b200_sample_chunked": [native.c_void_p, native.c_int, native.c_int, native.c_void_p, native.c_void_p,
                                native.c_int, native.c_int, native.c_void_p, native.c_int, native.c_void_p],
        "b200_sample_slots": [native.c_void_p, native.c_int, native.c_int, native.c_void_p, native.c_void_p, native.c_void_p,
                              native.c_int, native.c_int, native.c_void_p, native.c_int, native.c_void_p],
    },
)

CHUNKS = 64   # parts a row's vocabulary is cut into for the one-pass selections

PARAM_WORDS = 6
_MASK64 = (1 << 64) - 1


def fresh_seed() -> int:
    """A seed for a request that gave none (the reference falls back to the
    global generator there, mini_llm/sampling.py:94-101)."""

    return random.SystemRandom().getrandbits(63)


def _float_bits(value: float) -> int:
    return struct.unpack("<i", struct.pack("<f", value))[0]


def pack_row(config: SamplingConfig, seed: int, counter: int) -> list[int]:
    """[temperature bits, top_k (0: off), top_p bits, seed low, seed high, counter] as int32."""

    def s32(v: int) -> int:
        v &= 0xFFFFFFFF
        return v - (1 << 32) if v >= (1 << 31) else v

    return [
        _float_bits(config.temperature), config.top_k or 0, _float_bits(config.top_p),
        s32(seed), s32(seed >> 32), s32(counter),
    ]


class Sampler:
    """Greedy, temperature, top-k and top-p selection in one kernel launch for
    the whole batch; only the chosen token ids come back to the host."""

    def __init__(self, device: torch.device, max_rows: int = 256) -> None:
        self.device = device
        self._host = torch.empty(max_rows * PARAM_WORDS, dtype=torch.int32, pin_memory=True)
        self._dev = torch.empty(max_rows * PARAM_WORDS, dtype=torch.int32, device=device)
        self._out = torch.empty(max_rows, dtype=torch.int32, device=device)
        self._out_host = torch.empty(max_rows, dtype=torch.int32, pin_memory=True)
        self._scratch = torch.empty(max_rows * CHUNKS * 2, dtype=torch.int32, device=device)
        self.max_rows = max_rows

    def sample(self, logits: torch.Tensor, rows: Sequence[tuple[SamplingConfig, int, int]]) -> list[int]:
        """``rows[i] = (options, seed, counter)`` for ``logits[i]``; ``counter`` is the
        index of the token being generated for that request."""

        native.require(logits, "logits", dtype=torch.float32, dims=2)
        n, vocab = logits.shape
        if n != len(rows):
            raise SamplingError(f"{n} rows of logits but {len(rows)} sampling rows")
        if n > self.max_rows:
            raise SamplingError(f"at most {self.max_rows} rows can be sampled at once")
        for config, _, _ in rows:
            if config.top_k is not None and config.top_k > vocab:
                raise SamplingError(f"top_k {config.top_k} exceeds vocabulary size {vocab}")
        packed = np.asarray([w for config, seed, counter in rows for w in pack_row(config, seed, counter)], dtype=np.int32)
        self._host[: packed.shape[0]].numpy()[:] = packed
        self._dev[: packed.shape[0]].copy_(self._host[: packed.shape[0]], non_blocking=True)
        filtered = any(c.temperature > 0 and ((c.top_k is not None and c.top_k < vocab) or c.top_p < 1.0)
                       for c, _, _ in rows)
        chunks = CHUNKS if vocab >= 4096 else 1
        native.call("b200_sample_chunked", logits.data_ptr(), logits.stride(0), vocab, self._dev.data_ptr(),
                    self._out.data_ptr(), n, chunks, self._scratch.data_ptr(), 1 if filtered else 0,
                    native.stream_ptr(), launches=3 if filtered else 2)
        self._out_host[:n].copy_(self._out[:n], non_blocking=True)
        torch.cuda.current_stream(self.device).synchronize()
        tokens = self._out_host[:n].tolist()
        if any(t < 0 for t in tokens):
            raise SamplingError("logits must contain only finite values")
        return tokens

    def sample_slots(self, logits: torch.Tensor, records: torch.Tensor, row_slots: torch.Tensor, out: torch.Tensor, *,
                     filtered: bool) -> None:
        """Draw one token per row of ``logits`` with the options, seed and counter found in
        the slot record ``records[row_slots[i]]``, write it into ``out[i]`` and, with the
        advanced counter, back into the record.  Nothing is copied to the host and nothing
        waits: the call may sit inside a CUDA-graph capture.  ``filtered``: some row uses
        top-k or top-p (then the kernel for those rows runs too)."""

        native.require(logits, "logits", dtype=torch.float32, dims=2)
        n, vocab = logits.shape
        native.require(records, "records", dtype=torch.int32, dims=2)
        native.require(row_slots, "row_slots", dtype=torch.int32, shape=(n,))
        native.require(out, "out", dtype=torch.int32, dims=1)
        if n > self.max_rows or out.shape[0] < n:
            raise SamplingError(f"at most {min(self.max_rows, out.shape[0])} rows can be sampled at once")
        chunks = CHUNKS if vocab >= 4096 else 1
        native.call("b200_sample_slots", logits.data_ptr(), logits.stride(0), vocab, records.data_ptr(), row_slots.data_ptr(),
                    out.data_ptr(), n, chunks, self._scratch.data_ptr(), 1 if filtered else 0, native.stream_ptr(),
                    launches=3 if filtered else 2)
