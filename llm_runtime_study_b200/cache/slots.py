"""Per-request slot records: fixed-size state of every live request, on the device,
with a host mirror.

The reference keeps a request's position, its last sampled token, the index of the next
token and its random generator on the host (mini_llm/cache/lengths.py:8-43,
mini_llm/generation.py:56-70, mini_llm/sampling.py:94-101) and sends token ids and
positions to the device for every decode step (mini_llm/generation.py:251-255,
mini_llm/model/base.py:229-231).  Here a request's slot holds them on the device: the
decode step reads its token and position out of the record and advances the position,
the sampling kernels read their options, seed and counter there and write the chosen
token and the advanced counter back.  A decode step then needs from the host only the
list of slots in the batch and the block tables.

Layout of a record (int32 words; ``csrc/slots.h`` is the device's copy of it):
position, last token, temperature bits, top_k (0: off), top_p bits, seed low, seed
high, counter, live flag, three spare words.  The table has one record more than there
are request slots: the last belongs to nobody and is where the rows that pad a batch up
to the size of its captured graph point (never live, so those rows have length 0).

The host mirror is what the host *knows* without asking the device: everything but the
last token, which travels back with each step's sampled ids.
"""

from __future__ import annotations

import struct
from dataclasses import dataclass

import numpy as np
import torch

SLOT_WORDS = 12
POSITION, LAST_TOKEN, TEMPERATURE, TOP_K, TOP_P, SEED_LOW, SEED_HIGH, COUNTER, LIVE = range(9)


def _float_bits(value: float) -> int:
    return struct.unpack("<i", struct.pack("<f", value))[0]


def _s32(value: int) -> int:
    value &= 0xFFFFFFFF
    return value - (1 << 32) if value >= (1 << 31) else value


@dataclass(frozen=True)
class SlotRecord:
    """What the host writes into a slot: where the request stands and how it samples."""

    position: int            # tokens in the cache once the step that carries this record has run
    temperature: float = 0.0
    top_k: int = 0           # 0: off
    top_p: float = 1.0
    seed: int = 0
    counter: int = 0         # index of the next token to draw
    last_token: int = 0

    def words(self) -> list[int]:
        return [
            self.position, self.last_token, _float_bits(self.temperature), self.top_k, _float_bits(self.top_p),
            _s32(self.seed), _s32(self.seed >> 32), _s32(self.counter), 1, 0, 0, 0,
        ]

    @property
    def filtered(self) -> bool:
        """Whether drawing a token needs the top-k / top-p pass."""

        return self.temperature > 0 and (self.top_k > 0 or self.top_p < 1.0)


class SlotTable:
    def __init__(self, num_slots: int, device: torch.device) -> None:
        self.num_slots = num_slots
        self.padding_slot = num_slots
        self.records = torch.zeros((num_slots + 1, SLOT_WORDS), dtype=torch.int32, device=device)
        self.mirror = np.zeros((num_slots + 1, SLOT_WORDS), dtype=np.int32)

    def note(self, slot: int, record: SlotRecord) -> np.ndarray:
        """Remember on the host what is being written into ``slot``; return the words to write."""

        if not 0 <= slot < self.num_slots:
            raise IndexError(f"slot {slot} is not one of the {self.num_slots} request slots")
        self.mirror[slot] = record.words()
        return self.mirror[slot]

    def advanced(self, slot: int, *, tokens: int = 1, draws: int = 1) -> None:
        """The device fed ``tokens`` tokens of this slot and drew ``draws`` new ones."""

        self.mirror[slot, POSITION] += tokens
        self.mirror[slot, COUNTER] += draws

    def clear(self, slot: int) -> None:
        self.mirror[slot] = 0

    def filtered(self, slot: int) -> bool:
        row = self.mirror[slot]
        temperature = struct.unpack("<f", struct.pack("<i", int(row[TEMPERATURE])))[0]
        top_p = struct.unpack("<f", struct.pack("<i", int(row[TOP_P])))[0]
        return temperature > 0 and (int(row[TOP_K]) > 0 or top_p < 1.0)
