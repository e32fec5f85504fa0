"""Kernels over the per-request slot records (csrc/slots.cu)."""

from __future__ import annotations

import torch

from . import native
from .native import c_int, c_void_p

native.register_library(
    "b200_slots", ("slots.cu",),
    {
        "b200_slot_words": [],
        "b200_slot_store": [c_void_p, c_void_p, c_void_p, c_int, c_void_p],
        "b200_slot_load": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p],
    },
)


def slot_store(records: torch.Tensor, staged: torch.Tensor, slots: torch.Tensor) -> None:
    """``records[slots[i]] = staged[i]``."""

    native.require(records, "records", dtype=torch.int32, dims=2)
    native.require(slots, "slots", dtype=torch.int32, dims=1)
    native.require(staged, "staged", dtype=torch.int32, shape=(slots.shape[0], records.shape[1]))
    native.call("b200_slot_store", records.data_ptr(), staged.data_ptr(), slots.data_ptr(), slots.shape[0], native.stream_ptr())


def slot_load(records: torch.Tensor, slots: torch.Tensor, token_ids: torch.Tensor, positions: torch.Tensor,
              kv_len: torch.Tensor) -> None:
    """Fill a decode batch's token ids, positions and lengths from the records of its slots and
    advance the records' positions."""

    native.require(records, "records", dtype=torch.int32, dims=2)
    n = slots.shape[0]
    for t, name in ((slots, "slots"), (token_ids, "token_ids"), (positions, "positions"), (kv_len, "kv_len")):
        native.require(t, name, dtype=torch.int32, shape=(n,))
    native.call("b200_slot_load", records.data_ptr(), slots.data_ptr(), token_ids.data_ptr(), positions.data_ptr(),
                kv_len.data_ptr(), n, native.stream_ptr())
