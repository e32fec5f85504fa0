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

from dataclasses import dataclass, replace
from typing import Any, Sequence

import numpy as np
import torch

from ..cache.manager import CacheManager, RequestCache
from ..cache.slots import SLOT_WORDS, SlotRecord
from ..errors import GenerationError, KVCacheError, SamplingError
from ..ops import attention as attention_ops
from ..parts.base import Runtime


@dataclass
class StepEntry:
    """The next tokens of one request.  ``want`` lists the places among these
    tokens (0-based) whose logits are asked for; it may be empty.  ``sample``
    (``step_sampled`` only): draw the request's next token on the device from the
    logits at the entry's last token, with these options, and keep it in the
    request's slot record; ``want`` is then that one place."""

    request: RequestCache
    tokens: Sequence[int]
    want: Sequence[int] = ()
    sample: SlotRecord | None = None


class TokenHandle:
    """Token ids drawn on the device by a step, on their way to the host.  The
    step that produced them may still be running; ``tokens()`` waits for it."""

    def __init__(self, host: torch.Tensor, event: "torch.cuda.Event | None", count: int) -> None:
        self._host, self._event, self.count = host, event, count

    def tokens(self) -> list[int]:
        if self._event is not None:
            self._event.synchronize()
            self._event = None
        ids = self._host[: self.count].tolist()
        if any(t < 0 for t in ids):
            raise SamplingError("logits must contain only finite values")
        return ids


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
        self.logits_at_every_row = False         # the wanted rows are all rows, in order
        self.live_parts: Any = None              # under a graph capture: how the decode attention finds its parts per replay
        self.row_slots: torch.Tensor = None      # [M] int32 slot of each sampled row (step_sampled / decode_sampled)
        self.staged_records: torch.Tensor = None # [M, SLOT_WORDS] int32 records the host writes for the sampled rows

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
        self.last_logits: torch.Tensor | None = None   # logits of the last sampled step (valid until the next step)
        cuda = runtime.device.type == "cuda"
        rows = max(manager.max_requests, 1)
        self._ids_device = torch.zeros(rows, dtype=torch.int32, device=runtime.device)
        self._ids_host = [torch.zeros(rows, dtype=torch.int32, pin_memory=cuda) for _ in range(4)]
        self._ids_events: list[torch.cuda.Event | None] = [None] * 4
        self._ids_turn = 0

    # ---------------------------------------------------------------- build
    def build_context(self, entries: Sequence[StepEntry], *, table_width: int | None = None) -> StepContext:
        """Validate the batch on the host, take the pages it needs, and put its
        metadata on the device.  Nothing is launched and no length changes."""

        q_lens, starts = self.validate_and_grow(entries)
        manager = self.manager
        return self._pack_context(entries, q_lens, starts, table_width)

    def validate_and_grow(self, entries: Sequence[StepEntry], *, tokens_on_device: bool = False) -> tuple[list[int], list[int]]:
        """``tokens_on_device``: every entry is one decoded token that the device holds in
        the request's slot record (it came out of the sampler, so it is in the vocabulary)."""

        if not entries:
            raise GenerationError("a step needs at least one entry")
        manager = self.manager
        seen: set[int] = set()
        q_lens, starts = [], []
        for entry in entries:
            n = 1 if tokens_on_device else len(entry.tokens)
            if n == 0:
                raise GenerationError("an entry needs at least one token")
            if entry.request.released:
                raise KVCacheError("the request's cache has been released")
            if entry.request.id in seen:
                raise GenerationError("a request may appear once in a step")
            seen.add(entry.request.id)
            for t in (() if tokens_on_device else entry.tokens):
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
            if entry.sample is not None and list(entry.want) != [n - 1]:
                raise GenerationError("an entry whose next token is drawn on the device wants the logits of its last token only")
            if tokens_on_device and start == 0:
                raise GenerationError("a request with nothing in the cache has no decoded token to continue from")
            q_lens.append(n)
            starts.append(start)
        # pages for every entry, or for none: check the total first
        budget = manager.budget()
        for entry, start, n in zip(entries, starts, q_lens):
            held = manager.held(entry.request)
            if not budget.take(held, start + n):
                need, free = budget.short_by(held, start + n)
                raise KVCacheError(f"KV page pool exhausted: need {need} pages but only {free} are free")
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

        sampled = [e for e in entries if e.sample is not None]
        row_slots = np.asarray([e.request.slot for e in sampled], dtype=np.int32)
        staged = np.zeros((len(sampled), SLOT_WORDS), dtype=np.int32)
        for e, length in zip(entries, kv_lens):
            if e.sample is not None:    # the record's position is where the drawn token will go: the length after this step
                e.sample = replace(e.sample, position=length)
        for i, e in enumerate(sampled):
            staged[i] = manager.slots.note(e.request.slot, e.sample)
        pieces = [token_ids, positions, token_entry, q_start, np.asarray(kv_lens, dtype=np.int32), slots,
                  logit_rows, *[t.reshape(-1) for t in tables], row_slots, staged.reshape(-1)]
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
        ctx.row_slots = view(7 + len(tables))
        ctx.staged_records = view(8 + len(tables)).view(len(sampled), SLOT_WORDS)
        ctx.q_lens, ctx.kv_lens = q_lens, kv_lens
        ctx.entry_slots = [e.request.slot for e in entries]
        ctx.max_q_len, ctx.max_kv_len = max(q_lens), max(kv_lens)
        ctx.all_decode = ctx.max_q_len == 1
        ctx.logits_at_every_row = logit_rows.shape[0] == num_tokens and bool((logit_rows == np.arange(num_tokens)).all())
        return ctx

    # ------------------------------------------------------------------ run
    def step(self, entries: Sequence[StepEntry]) -> torch.Tensor | None:
        """Run one batch.  Returns float32 logits ``[wanted, vocab]`` on the
        device, rows in the order of the entries and of each entry's ``want``
        (``None`` if nothing was wanted).  The tensor is the caller's."""

        ctx = self.build_context(entries)
        with torch.inference_mode():
            logits = self.model.forward(ctx)
        for entry, length in zip(entries, ctx.kv_lens):
            self.manager.commit(entry.request, length)
        self.last_context = ctx
        return logits

    # ------------------------------------------- steps that draw on the device
    def _send_home(self, ids: torch.Tensor, count: int) -> TokenHandle:
        """Start the copy of ``count`` drawn ids into pinned host memory; do not wait."""

        self._ids_turn = (self._ids_turn + 1) % len(self._ids_host)
        event = self._ids_events[self._ids_turn]
        if event is not None:
            event.synchronize()          # the host has long read what this buffer held four steps ago
        host = self._ids_host[self._ids_turn]
        host[:count].copy_(ids[:count], non_blocking=True)
        if self.runtime.device.type != "cuda":
            return TokenHandle(host, None, count)
        event = event or torch.cuda.Event()
        event.record()
        self._ids_events[self._ids_turn] = event
        return TokenHandle(host, event, count)

    def step_sampled(self, entries: Sequence[StepEntry], sampler: Any) -> TokenHandle | None:
        """Run one batch packed by the host (prompt portions, decoded tokens whose ids the
        host knows) and draw, on the device, the next token of every entry that carries a
        ``sample`` record.  The records are written into the requests' slots before the
        draw; afterwards each slot holds the drawn token and the advanced counter, so the
        request can go on with ``decode_sampled`` without the host.  Returns the handle of
        the drawn ids (in the order of the sampled entries), or ``None`` if none is drawn."""

        from ..ops import slots as slot_ops

        ctx = self.build_context(entries)
        sampled = [e for e in entries if e.sample is not None]
        with torch.inference_mode():
            if sampled:
                slot_ops.slot_store(self.manager.slots.records, ctx.staged_records, ctx.row_slots)
            logits = self.model.forward(ctx)
            if sampled:
                sampler.sample_slots(logits, self.manager.slots.records, ctx.row_slots, self._ids_device,
                                     filtered=any(e.sample.filtered for e in sampled))
        for entry, length in zip(entries, ctx.kv_lens):
            self.manager.commit(entry.request, length)
        for entry in sampled:
            self.manager.slots.advanced(entry.request.slot, tokens=0, draws=1)
        self.last_context, self.last_logits = ctx, logits
        return self._send_home(self._ids_device, len(sampled)) if sampled else None

    def decode_sampled(self, requests: Sequence[RequestCache], sampler: Any) -> TokenHandle:
        """One decode step for requests whose pending token is in their slot records: feed
        it, draw the next one, keep it in the record.  Nothing but the list of slots and the
        block tables goes to the device, and nothing but the drawn ids comes back.  With
        ``use_cuda_graph`` the step (embedding to sampling) is replayed from a CUDA graph
        whenever every part of the model allows it."""

        entries = [StepEntry(r, (), [0]) for r in requests]
        self.validate_and_grow(entries, tokens_on_device=True)
        filtered = any(self.manager.slots.filtered(r.slot) for r in requests)
        use_graph = (self.use_cuda_graph and self.runtime.device.type == "cuda"
                     and getattr(self.model, "graph_safe", lambda: False)())
        if use_graph:
            if self._graphs is None:
                from .graph import DecodeGraphs

                self._graphs = DecodeGraphs(self)
            ids, self.last_logits = self._graphs.run(requests, sampler, filtered)
        else:
            ids, self.last_logits = self._decode_eager(requests, sampler, filtered)
        for request in requests:
            self.manager.commit(request, request.length + 1)
            self.manager.slots.advanced(request.slot, tokens=1, draws=1)
        return self._send_home(ids, len(requests))

    def _decode_eager(self, requests: Sequence[RequestCache], sampler: Any, filtered: bool):
        """The launches a captured decode step holds, issued one by one."""

        from ..ops import slots as slot_ops

        manager = self.manager
        n = len(requests)
        starts = [r.length for r in requests]
        tables = []
        for g in range(len(manager.layout.groups)):
            width = _round_up(max(max(len(r.tables[g]) for r in requests), 1), 4)
            table = np.full((n, width), -1, dtype=np.int32)
            for i, r in enumerate(requests):
                table[i, : len(r.tables[g])] = r.tables[g]
            tables.append(table)
        ramp = np.arange(n + 1, dtype=np.int32)
        slots = np.asarray([r.slot for r in requests], dtype=np.int32)
        blank = np.zeros(n, dtype=np.int32)
        # token ids, positions and lengths are filled in on the device from the slot records
        pieces = [blank, blank, ramp[:n], ramp, blank, slots, ramp[:n], *[t.reshape(-1) for t in tables]]
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
        ctx.num_tokens = ctx.num_entries = ctx.num_logit_rows = n
        ctx.token_ids, ctx.positions, ctx.token_entry = view(0), view(1), view(2)
        ctx.q_start, ctx.kv_len, ctx.slots, ctx.logit_rows = view(3), view(4), view(5), view(6)
        ctx.tables = [view(7 + g).view(n, tables[g].shape[1]) for g in range(len(tables))]
        ctx.row_slots = ctx.slots
        ctx.q_lens, ctx.kv_lens = [1] * n, [s + 1 for s in starts]
        ctx.entry_slots = [r.slot for r in requests]
        ctx.max_q_len, ctx.max_kv_len = 1, max(ctx.kv_lens)
        ctx.all_decode = ctx.logits_at_every_row = True
        with torch.inference_mode():
            slot_ops.slot_load(manager.slots.records, ctx.slots, ctx.token_ids, ctx.positions, ctx.kv_len)
            logits = self.model.forward(ctx)
            sampler.sample_slots(logits, manager.slots.records, ctx.row_slots, self._ids_device, filtered=filtered)
        self.last_context = ctx
        return self._ids_device, logits
