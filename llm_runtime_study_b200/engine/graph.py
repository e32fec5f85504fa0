"""CUDA-graph replay of the decode step.

The reference captures the decoder stack once per batch size over a block table of
fixed width and leaves the output head and the sampling outside
(mini_llm/cuda_graph.py:89-187).  Here the whole step is captured, from the reading of
the requests' slot records (token, position) through the layers and the output head to
the sampling kernels that write the drawn token back into the records.  One graph per

* batch-size *bucket* (1, 2, 4, 8, ... and the largest batch): a batch is padded up to
  its bucket with rows that point at the padding slot, which is never live (length 0,
  no pages: the cache-write and the attention kernels skip them), so a batch that
  shrinks or grows by one does not pay a new capture;
* whether some row needs the top-k / top-p pass of the sampler.

Kernels launched under capture size their grids from an upper bound of the sequence
lengths that cannot change afterwards (the longest sequence the engine was opened for).
The decode attention still cuts a replay's sequences into the number of parts that
suits them: with the step's other inputs the host sends, for every kind of attention
launch in the graph, how many of its grid's parts this batch's longest sequence needs
(``ops/attention_bf16.LiveParts``); the CTAs of the other parts leave at once.

All per-step input lives in one persistent device buffer whose layout is fixed by the
bucket and the table width: the slots of the batch, the numbers of parts, the block tables.  It is copied
only when it differs from what the device already holds, so a replay is at most one
host-to-device copy plus one graph launch.  Graphs share one memory pool: they run one
after the other on one stream, and what leaves a graph (the drawn ids) lies outside it.
Steps that hold prompt portions run eagerly.
"""

from __future__ import annotations

import gc
from typing import Any, Sequence

import numpy as np
import torch

from ..cache.manager import RequestCache
from .step import StepContext, _round_up


LIVE_PLACES = 8      # kinds of decode attention launches (geometries) a captured step may hold


class DecodeGraph:
    """One captured decode step for exactly ``batch`` rows."""

    def __init__(self, owner: "DecodeGraphs", batch: int, filtered: bool) -> None:
        runner = owner.runner
        self.runner, self.batch, self.filtered = runner, batch, filtered
        manager = runner.manager
        self.bound = manager.max_seq_len
        # a block table wide enough for the longest sequence, per group (groups may differ in page size)
        self.table_widths = [_round_up(-(-manager.max_seq_len // pool.page_size), 4) for pool in manager.groups]
        self.groups = len(manager.layout.groups)
        b = batch
        # what the host sends every step (slots, numbers of parts, tables), then what never changes, then what the device fills in
        sizes = [b, LIVE_PLACES] + [b * w for w in self.table_widths] + [b, b + 1, b] + [b, b, b]
        self.offsets, total = [], 0
        for size in sizes:
            self.offsets.append(total)
            total += _round_up(size, 4)
        self.sizes = sizes
        self.sent = self.offsets[2 + self.groups]          # words copied per step
        device = runner.runtime.device
        self.dev = torch.zeros(total, dtype=torch.int32, device=device)
        self.host = [torch.zeros(self.sent, dtype=torch.int32, pin_memory=True) for _ in range(2)]
        self.events: list[torch.cuda.Event | None] = [None, None]
        self.turn = 0
        self.on_device: np.ndarray | None = None           # what the device holds of the sent part
        self.always_send = False                            # copy even what has not changed (measurements)
        self.graph: torch.cuda.CUDAGraph | None = None
        self.logits: torch.Tensor | None = None
        self.kernel_launches = 0
        ramp = torch.arange(b + 1, dtype=torch.int32, device=device)
        g = self.groups
        self._view(2 + g).copy_(ramp[:b])                   # token -> entry
        self._view(3 + g).copy_(ramp)                       # first token of each entry
        self._view(4 + g).copy_(ramp[:b])                   # rows whose logits are wanted: all
        self.ctx = self._static_context()

    def _view(self, i: int) -> torch.Tensor:
        return self.dev[self.offsets[i] : self.offsets[i] + self.sizes[i]]

    def _static_context(self) -> StepContext:
        runner, b, g = self.runner, self.batch, self.groups
        ctx = StepContext(runner.runtime, runner.manager)
        ctx.num_tokens = ctx.num_entries = ctx.num_logit_rows = b
        from ..ops.attention_bf16 import LiveParts

        ctx.slots = ctx.row_slots = self._view(0)
        ctx.live_parts = LiveParts(self._view(1), self.bound)
        ctx.tables = [self._view(2 + i).view(b, self.table_widths[i]) for i in range(g)]
        ctx.token_entry, ctx.q_start, ctx.logit_rows = self._view(2 + g), self._view(3 + g), self._view(4 + g)
        ctx.token_ids, ctx.positions, ctx.kv_len = self._view(5 + g), self._view(6 + g), self._view(7 + g)
        ctx.q_lens = [1] * b
        # kernels launched under capture may only size their grids from limits that never change
        ctx.kv_lens = [self.bound] * b
        ctx.max_q_len, ctx.max_kv_len = 1, self.bound
        ctx.all_decode = ctx.logits_at_every_row = True
        ctx.captured = True
        ctx.entry_slots = None     # the slots of a replay are on the device only (``ctx.slots``)
        return ctx

    def _fill(self, requests: Sequence[RequestCache]) -> None:
        """This step's slots and block tables.  Rows beyond the requests are padding: the
        slot that is never live and an empty block table."""

        b = self.batch
        manager = self.runner.manager
        sent = np.full(self.sent, -1, dtype=np.int32)
        sent[:b] = manager.padding_slot
        sent[: len(requests)] = [r.slot for r in requests]
        sent[b : self.offsets[2]] = 0
        parts = self.ctx.live_parts.fill(max(r.length for r in requests) + 1)    # for the longest sequence once this step has run
        sent[self.offsets[1] : self.offsets[1] + len(parts)] = parts
        for g in range(self.groups):
            o, w = self.offsets[2 + g], self.table_widths[g]
            table = sent[o : o + b * w].reshape(b, w)
            for i, r in enumerate(requests):
                row = r.tables[g]
                table[i, : len(row)] = row
        if self.on_device is not None and not self.always_send and np.array_equal(sent, self.on_device):
            return
        self.turn ^= 1
        event = self.events[self.turn]
        if event is not None:
            event.synchronize()
        self.host[self.turn].numpy()[:] = sent
        self.dev[: self.sent].copy_(self.host[self.turn], non_blocking=True)
        event = event or torch.cuda.Event()
        event.record()
        self.events[self.turn] = event
        self.on_device = sent

    def _launches(self, sampler: Any, ids: torch.Tensor) -> torch.Tensor:
        from ..ops import slots as slot_ops

        records = self.runner.manager.slots.records
        ctx = self.ctx
        slot_ops.slot_load(records, ctx.slots, ctx.token_ids, ctx.positions, ctx.kv_len)
        logits = self.runner.model.forward(ctx)
        sampler.sample_slots(logits, records, ctx.row_slots, ids, filtered=self.filtered)
        return logits

    def capture(self, sampler: Any, ids: torch.Tensor, pool: Any) -> None:
        """Capture the step.  Called with this step's slots and tables already in place, so
        that the run before the capture (library handles, workspaces) is an ordinary step;
        it is undone afterwards: the slot records (positions, counters) and the mixers'
        fixed-size state are put back, and the rows it wrote into the paged cache are
        written again, identically, by the replay."""

        from ..ops import native

        manager = self.runner.manager
        records = manager.slots.records
        saved = records.clone()
        saved_states = {layer: state.clone() for layer, state in manager.state_arrays.items()}
        stream = torch.cuda.Stream(device=self.runner.runtime.device)
        stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(stream), torch.inference_mode():
            self._launches(sampler, ids)
            records.copy_(saved)
            for layer, state in saved_states.items():
                manager.state_arrays[layer].copy_(state)
        torch.cuda.current_stream().wait_stream(stream)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        before = native.launch_count()
        # Nothing may be destroyed on the device while the stream is capturing: unreachable objects of earlier
        # engines (their graphs, their tensors) go now, and the collector stays off until the capture has ended.
        gc.collect()
        collecting = gc.isenabled()
        gc.disable()
        try:
            with torch.inference_mode(), torch.cuda.graph(graph, pool=pool):
                self.logits = self._launches(sampler, ids)
        finally:
            if collecting:
                gc.enable()
        self.kernel_launches = native.launch_count() - before
        native.add_launches(-self.kernel_launches)   # capturing launched nothing
        self.graph = graph

    def run(self, requests: Sequence[RequestCache], sampler: Any, ids: torch.Tensor, pool: Any) -> torch.Tensor:
        from ..ops import native

        self._fill(requests)
        if self.graph is None:
            self.capture(sampler, ids, pool)
            self._fill(requests)      # the attention launches have said by now what they need to be told
        self.graph.replay()
        native.add_launches(self.kernel_launches)
        return self.logits[: len(requests)]


class DecodeGraphs:
    """Graphs by (batch-size bucket, filtered), captured on first use."""

    def __init__(self, runner: Any) -> None:
        self.runner = runner
        self._graphs: dict[tuple[int, bool], DecodeGraph] = {}
        self._pool = None

    def bucket(self, batch: int) -> int:
        """The smallest power of two that holds the batch, but never more rows than
        the cache has request slots."""

        size = 1
        while size < batch:
            size *= 2
        return max(batch, min(size, self.runner.manager.max_requests))

    def graph_for(self, batch: int) -> DecodeGraph | None:
        """Some captured graph of the bucket that holds ``batch`` rows (for reports)."""

        size = self.bucket(batch)
        return next((g for (b, _), g in self._graphs.items() if b == size), None)

    def run(self, requests: Sequence[RequestCache], sampler: Any, filtered: bool) -> tuple[torch.Tensor, torch.Tensor]:
        """Replay the step for these requests; returns (drawn ids on the device, logits).
        Both belong to the graphs: they are valid until the next step."""

        runner = self.runner
        if self._pool is None:
            self._pool = torch.cuda.graph_pool_handle()
        key = (self.bucket(len(requests)), bool(filtered))
        graph = self._graphs.get(key)
        if graph is None:
            graph = self._graphs[key] = DecodeGraph(self, *key)
        logits = graph.run(requests, sampler, runner._ids_device, self._pool)
        return runner._ids_device, logits
