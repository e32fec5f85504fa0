"""The step function: one batch of (request, its next tokens) in, logits at the
wanted places out.

The reference has two entry points: ``prefill`` for one whole prompt and
``decode`` for one token of each of B requests (mini_llm/model/base.py:161-248).
Here there is one: a batch holds, for each request in it, the next ``n >= 1``
tokens; a portion of a prompt cut anywhere sits beside single decoded tokens.
Only the tokens given are run; everything before them comes from the cache.
Activations are flat ``[tokens, width]``; per-token metadata (position, which
entry) and per-entry metadata (block-table row, lengths) go to the device in one
copy.  Lengths are committed after the launches succeeded; an exception leaves
them as they were (the reference extends first and rolls back on failure,
mini_llm/model/base.py:175, 188-190: the same contract seen from outside).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Sequence

import numpy as np
import torch

from ..cache.manager import CacheManager, RequestCache
from ..errors import GenerationError, KVCacheError
from ..ops import attention as attention_ops
from ..parts.base import Runtime


@dataclass
class StepEntry:
    """The next tokens of one request.  ``want`` lists the places among these
    tokens (0-based) whose logits are asked for; it may be empty."""

    request: RequestCache
    tokens: Sequence[int]
    want: Sequence[int] = ()


class StepContext:
    """Everything a part may read about the batch being run."""

    def __init__(self, runtime: Runtime, manager: CacheManager) -> None:
        self.runtime = runtime
        self.manager = manager
        self.num_tokens = 0
        self.num_entries = 0
        self.num_logit_rows = 0
        self.token_ids: torch.Tensor = None      # [N] int32
        self.positions: torch.Tensor = None      # [N] int32 absolute position of each token
        self.token_entry: torch.Tensor = None    # [N] int32 which entry (row) a token belongs to
        self.q_start: torch.Tensor = None        # [R+1] int32 first token of each entry
        self.kv_len: torch.Tensor = None         # [R] int32 length of each request after this step
        self.slots: torch.Tensor = None          # [R] int32 request slot of each entry
        self.logit_rows: torch.Tensor = None     # [M] int32 rows whose logits are wanted
        self.tables: list[torch.Tensor] = []     # per page group: [R, width] int32
        # host-side copies, for choosing kernels and grids
        self.q_lens: list[int] = []
        self.kv_lens: list[int] = []
        self.entry_slots: list[int] = []
        self.max_q_len = 0
        self.max_kv_len = 0
        self.all_decode = False
        self.captured = False   # True while a CUDA graph holds this batch's launches

    def block_table(self, group: int) -> torch.Tensor:
        return self.tables[group]

    def attention(self, q: torch.Tensor, cache: Any, *, scale: float, window: int = 0) -> torch.Tensor:
        return attention_ops.paged_attention(q, cache, self, scale=scale, window=window)


class _MetaBuffers:
    """A small ring of pinned host buffers and one device buffer for the step's
    integer metadata, so that a step costs one host-to-device copy."""

    RING = 4

    def __init__(self, device: torch.device, capacity: int) -> None:
        self.device = device
        self.capacity = 0
        self.host: list[torch.Tensor] = []
        self.events: list[torch.cuda.Event | None] = []
        self.dev: torch.Tensor | None = None
        self.turn = 0
        self._reserve(capacity)

    def _reserve(self, capacity: int) -> None:
        if capacity <= self.capacity:
            return
        if self.device.type == "cuda":
            torch.cuda.current_stream(self.device).synchronize()
        self.capacity = capacity
        pin = self.device.type == "cuda"
        self.host = [torch.empty(capacity, dtype=torch.int32, pin_memory=pin) for _ in range(self.RING)]
        self.events = [None] * self.RING
        self.dev = torch.empty(capacity, dtype=torch.int32, device=self.device)

    def upload(self, packed: np.ndarray) -> torch.Tensor:
        n = packed.shape[0]
        self._reserve(max(n, 1))
        self.turn = (self.turn + 1) % self.RING
        event = self.events[self.turn]
        if event is not None:
            event.synchronize()
        host = self.host[self.turn]
        host[:n].numpy()[:] = packed
        dev = self.dev[:n]
        dev.copy_(host[:n], non_blocking=True)
        if self.device.type == "cuda":
            event = event or torch.cuda.Event()
            event.record()
            self.events[self.turn] = event
        return dev


def _round_up(value: int, multiple: int) -> int:
    return -(-value // multiple) * multiple


class StepRunner:
    """Runs batches through a model against a cache manager."""

    def __init__(self, model: Any, manager: CacheManager, runtime: Runtime, *, vocab_size: int, max_positions: int) -> None:
        self.model = model
        self.manager = manager
        self.runtime = runtime
        self.vocab_size = vocab_size
        self.max_positions = max_positions
        self._buffers = _MetaBuffers(runtime.device, 4096)
        model.bind_cache(manager)
        self.last_context: StepContext | None = None
        self.use_cuda_graph = False
        self._graphs = None

    # ---------------------------------------------------------------- build
    def build_context(self, entries: Sequence[StepEntry], *, table_width: int | None = None) -> StepContext:
        """Validate the batch on the host, take the pages it needs, and put its
        metadata on the device.  Nothing is launched and no length changes."""

        q_lens, starts = self.validate_and_grow(entries)
        manager = self.manager
        return self._pack_context(entries, q_lens, starts, table_width)

    def validate_and_grow(self, entries: Sequence[StepEntry]) -> tuple[list[int], list[int]]:
        if not entries:
            raise GenerationError("a step needs at least one entry")
        manager = self.manager
        seen: set[int] = set()
        q_lens, starts = [], []
        for entry in entries:
            n = len(entry.tokens)
            if n == 0:
                raise GenerationError("an entry needs at least one token")
            if entry.request.released:
                raise KVCacheError("the request's cache has been released")
            if entry.request.id in seen:
                raise GenerationError("a request may appear once in a step")
            seen.add(entry.request.id)
            for t in entry.tokens:
                if not 0 <= int(t) < self.vocab_size:
                    raise GenerationError(f"token id {t} is outside the vocabulary [0, {self.vocab_size})")
            start = entry.request.length
            if start + n > self.max_positions:
                raise GenerationError(
                    f"position {start + n - 1} exceeds the model limit {self.max_positions - 1}"
                )
            for w in entry.want:
                if not 0 <= int(w) < n:
                    raise GenerationError(f"wanted place {w} is outside the entry's {n} tokens")
            q_lens.append(n)
            starts.append(start)
        # pages for every entry, or for none: check the total first
        for g, allocator in enumerate(manager.allocators):
            need = sum(
                max(0, -(-(s + n) // manager.page_size) - len(e.request.tables[g]))
                for e, s, n in zip(entries, starts, q_lens)
            )
            if need > allocator.num_free:
                raise KVCacheError(
                    f"KV page pool exhausted: need {need} pages but only {allocator.num_free} are free"
                )
        for entry, start, n in zip(entries, starts, q_lens):
            manager.grow(entry.request, start + n)
        return q_lens, starts

    def _pack_context(self, entries, q_lens, starts, table_width) -> StepContext:
        manager = self.manager
        num_tokens, num_entries = sum(q_lens), len(entries)
        token_ids = np.concatenate([np.asarray(e.tokens, dtype=np.int32) for e in entries])
        positions = np.concatenate([np.arange(s, s + n, dtype=np.int32) for s, n in zip(starts, q_lens)])
        token_entry = np.repeat(np.arange(num_entries, dtype=np.int32), q_lens)
        q_start = np.zeros(num_entries + 1, dtype=np.int32)
        np.cumsum(q_lens, out=q_start[1:])
        kv_lens = [s + n for s, n in zip(starts, q_lens)]
        slots = np.asarray([e.request.slot for e in entries], dtype=np.int32)
        logit_rows = np.asarray(
            [q_start[i] + int(w) for i, e in enumerate(entries) for w in e.want], dtype=np.int32
        )
        tables = []
        for g in range(len(manager.layout.groups)):
            width = max(len(e.request.tables[g]) for e in entries)
            width = table_width if table_width is not None else _round_up(max(width, 1), 4)
            table = np.full((num_entries, width), -1, dtype=np.int32)
            for i, e in enumerate(entries):
                row = e.request.tables[g]
                table[i, : len(row)] = row
            tables.append(table)

        pieces = [token_ids, positions, token_entry, q_start, np.asarray(kv_lens, dtype=np.int32), slots,
                  logit_rows, *[t.reshape(-1) for t in tables]]
        # every piece starts on a 16-byte boundary
        offsets, total = [], 0
        for piece in pieces:
            offsets.append(total)
            total += _round_up(piece.shape[0], 4)
        packed = np.zeros(total, dtype=np.int32)
        for piece, off in zip(pieces, offsets):
            packed[off : off + piece.shape[0]] = piece
        dev = self._buffers.upload(packed)

        def view(i: int) -> torch.Tensor:
            return dev[offsets[i] : offsets[i] + pieces[i].shape[0]]

        ctx = StepContext(self.runtime, manager)
        ctx.num_tokens, ctx.num_entries, ctx.num_logit_rows = num_tokens, num_entries, int(logit_rows.shape[0])
        ctx.token_ids, ctx.positions, ctx.token_entry = view(0), view(1), view(2)
        ctx.q_start, ctx.kv_len, ctx.slots, ctx.logit_rows = view(3), view(4), view(5), view(6)
        ctx.tables = [view(7 + g).view(num_entries, tables[g].shape[1]) for g in range(len(tables))]
        ctx.q_lens, ctx.kv_lens = q_lens, kv_lens
        ctx.entry_slots = [e.request.slot for e in entries]
        ctx.max_q_len, ctx.max_kv_len = max(q_lens), max(kv_lens)
        ctx.all_decode = ctx.max_q_len == 1
        return ctx

    # ------------------------------------------------------------------ run
    def step(self, entries: Sequence[StepEntry]) -> torch.Tensor | None:
        """Run one batch.  Returns float32 logits ``[wanted, vocab]`` on the
        device, rows in the order of the entries and of each entry's ``want``
        (``None`` if nothing was wanted)."""

        if self.use_cuda_graph and self.runtime.device.type == "cuda":
            if self._graphs is None:
                from .graph import DecodeGraphs

                self._graphs = DecodeGraphs(self)
            if self._graphs.eligible(entries):
                return self._step_captured(entries)
        ctx = self.build_context(entries)
        with torch.inference_mode():
            logits = self.model.forward(ctx)
        for entry, length in zip(entries, ctx.kv_lens):
            self.manager.commit(entry.request, length)
        self.last_context = ctx
        return logits

    def _step_captured(self, entries: Sequence[StepEntry]) -> torch.Tensor:
        """A batch of single decoded tokens, replayed from a CUDA graph.  The
        same host-side checks and page-taking as the eager path come first."""

        self.validate_and_grow(entries)
        logits, kv_lens = self._graphs.run(entries)
        for entry, length in zip(entries, kv_lens):
            self.manager.commit(entry.request, length)
        return logits
