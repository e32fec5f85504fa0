"""CUDA-graph replay of the pure-decode step.

The reference captures the decoder stack once per batch size over a block table
of fixed width and leaves the output head outside (mini_llm/cuda_graph.py:89-187).
Here the whole step is captured (embedding to logits) once per batch-size *bucket*
(1, 2, 4, 8, ... and the largest batch): a batch is padded up to its bucket with
rows that hold no request (length 0, no pages: the cache-write and the attention
kernels skip them), so a batch that shrinks or grows by one does not pay a new
capture.  All metadata lives in one persistent device buffer whose layout is fixed
by the bucket and the table width, so a replay is one host-to-device copy plus one
graph launch.  Steps that hold prompt portions run eagerly.
"""

from __future__ import annotations

from typing import Any, Sequence

import numpy as np
import torch

from .step import StepContext, StepEntry, _round_up


class DecodeGraph:
    """One captured decode step for exactly ``batch`` requests."""

    def __init__(self, runner: Any, batch: int) -> None:
        self.runner = runner
        self.batch = batch
        manager = runner.manager
        self.table_width = _round_up(-(-manager.max_seq_len // manager.page_size), 4)
        self.groups = len(manager.layout.groups)
        b, w = batch, self.table_width
        sizes = [b, b, b, b + 1, b, b, b] + [b * w] * self.groups
        self.offsets, total = [], 0
        for size in sizes:
            self.offsets.append(total)
            total += _round_up(size, 4)
        self.sizes = sizes
        device = runner.runtime.device
        self.dev = torch.zeros(total, dtype=torch.int32, device=device)
        self.host = [torch.zeros(total, dtype=torch.int32, pin_memory=True) for _ in range(2)]
        self.events: list[torch.cuda.Event | None] = [None, None]
        self.turn = 0
        self.graph: torch.cuda.CUDAGraph | None = None
        self.logits: torch.Tensor | None = None
        self.kernel_launches = 0
        self.ctx = self._static_context()

    def _view(self, i: int) -> torch.Tensor:
        return self.dev[self.offsets[i] : self.offsets[i] + self.sizes[i]]

    def _static_context(self) -> StepContext:
        runner, b = self.runner, self.batch
        ctx = StepContext(runner.runtime, runner.manager)
        ctx.num_tokens = ctx.num_entries = ctx.num_logit_rows = b
        ctx.token_ids, ctx.positions, ctx.token_entry = self._view(0), self._view(1), self._view(2)
        ctx.q_start, ctx.kv_len, ctx.slots, ctx.logit_rows = self._view(3), self._view(4), self._view(5), self._view(6)
        ctx.tables = [self._view(7 + g).view(b, self.table_width) for g in range(self.groups)]
        ctx.q_lens = [1] * b
        # kernels launched under capture may only size their grids from limits that never change
        ctx.kv_lens = [runner.manager.max_seq_len] * b
        ctx.max_q_len, ctx.max_kv_len = 1, runner.manager.max_seq_len
        ctx.all_decode = True
        ctx.captured = True
        return ctx

    def _fill(self, entries: Sequence[StepEntry]) -> list[int]:
        """Write this step's metadata into the persistent buffer.  Rows beyond the
        entries are padding: token 0 at position 0 of a sequence of length 0 whose block
        table is empty."""

        b, w = self.batch, self.table_width
        n = len(entries)
        self.turn ^= 1
        event = self.events[self.turn]
        if event is not None:
            event.synchronize()
        host = self.host[self.turn].numpy()
        starts = [e.request.length for e in entries]
        kv_lens = [s + 1 for s in starts]
        o = self.offsets
        pad = [0] * (b - n)
        host[o[0] : o[0] + b] = [int(e.tokens[0]) for e in entries] + pad
        host[o[1] : o[1] + b] = starts + pad
        host[o[2] : o[2] + b] = np.arange(b)
        host[o[3] : o[3] + b + 1] = np.arange(b + 1)
        host[o[4] : o[4] + b] = kv_lens + pad
        host[o[5] : o[5] + b] = [e.request.slot for e in entries] + pad
        host[o[6] : o[6] + b] = np.arange(b)
        for g in range(self.groups):
            table = host[o[7 + g] : o[7 + g] + b * w].reshape(b, w)
            table.fill(-1)
            for i, e in enumerate(entries):
                row = e.request.tables[g]
                table[i, : len(row)] = row
        self.dev.copy_(self.host[self.turn], non_blocking=True)
        event = event or torch.cuda.Event()
        event.record()
        self.events[self.turn] = event
        self.ctx.entry_slots = [e.request.slot for e in entries]
        return kv_lens

    def run(self, entries: Sequence[StepEntry]) -> tuple[torch.Tensor, list[int]]:
        from ..ops import native

        kv_lens = self._fill(entries)
        if self.graph is None:
            model = self.runner.model
            stream = torch.cuda.Stream(device=self.runner.runtime.device)
            stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(stream), torch.inference_mode():
                model.forward(self.ctx)          # warm-up outside capture (library handles, workspaces)
            torch.cuda.current_stream().wait_stream(stream)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            before = native.launch_count()
            with torch.inference_mode(), torch.cuda.graph(graph):
                self.logits = model.forward(self.ctx)
            self.kernel_launches = native.launch_count() - before
            native.add_launches(-self.kernel_launches)   # capturing launched nothing
            self.graph = graph
        self.graph.replay()
        native.add_launches(self.kernel_launches)
        return self.logits[: len(entries)], kv_lens


class DecodeGraphs:
    """Graphs by batch-size bucket, captured on first use."""

    def __init__(self, runner: Any) -> None:
        self.runner = runner
        self._graphs: dict[int, DecodeGraph] = {}

    def eligible(self, entries: Sequence[StepEntry]) -> bool:
        return all(len(e.tokens) == 1 and list(e.want) == [0] for e in entries)

    def bucket(self, batch: int) -> int:
        """The smallest power of two that holds the batch, but never more rows than
        the cache has request slots."""

        size = 1
        while size < batch:
            size *= 2
        return max(batch, min(size, self.runner.manager.max_requests))

    def run(self, entries: Sequence[StepEntry]) -> tuple[torch.Tensor, list[int]]:
        size = self.bucket(len(entries))
        graph = self._graphs.get(size)
        if graph is None:
            graph = self._graphs[size] = DecodeGraph(self.runner, size)
        return graph.run(entries)
