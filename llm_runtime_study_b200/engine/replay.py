"""Trace replay: feed given token ids through the model step by step and write
the logits.  It samples nothing and owns no forward pass, cache or loader: it
drives the same model, step function, cache manager and kernels as generation.

Input: one JSON object a line,
``{"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}``.
All entries of a step are one batch.  A request id seen for the first time
takes a slot; ids under ``end`` give back what they hold after the step.  For a
step in which something is wanted, ``<out>/<step>.f32`` receives the logits at
the wanted places, in the order of the entries and of ``want``, as little-endian
float32 ``[wanted, vocab]``.  After every step ``done <step>`` is printed.
"""

from __future__ import annotations

import json
import sys
from pathlib import Path
from typing import IO, Iterable

import numpy as np
import torch

from ..cache.manager import RequestCache
from ..errors import GenerationError
from .runtime import LoadedModel, load
from .step import StepEntry, StepRunner

DEFAULT_LIVE_REQUESTS = 16


class TraceReplayer:
    def __init__(self, loaded: LoadedModel, *, max_tokens: int, page_size: int = 16, out_dir: str | Path | None = None,
                 max_requests: int = DEFAULT_LIVE_REQUESTS) -> None:
        if max_tokens <= 0:
            raise GenerationError("--max-tokens must be positive")
        # The caller counts each request rounded up to a multiple of 64 tokens; a
        # page size that divides 64 never needs more pages than that count gives.
        if 64 % page_size and page_size % 64:
            raise GenerationError(f"page size {page_size} must divide 64 or be a multiple of it")
        self.loaded = loaded
        self.runner: StepRunner = loaded.make_runner(
            max_tokens=max_tokens, page_size=page_size, max_requests=max_requests
        )
        self.live: dict[str, RequestCache] = {}
        self.out_dir = None if out_dir is None else Path(out_dir)
        if self.out_dir is not None:
            self.out_dir.mkdir(parents=True, exist_ok=True)

    def run_step(self, record: dict) -> np.ndarray | None:
        """Run one step record; return the wanted logits ``[wanted, vocab]``
        (float32, host) or ``None``."""

        manager = self.runner.manager
        entries = []
        admitted: list[str] = []
        try:
            for item in record.get("entries", []):
                rid = str(item["id"])
                if rid not in self.live:
                    self.live[rid] = manager.admit()
                    admitted.append(rid)
                entries.append(StepEntry(self.live[rid], [int(t) for t in item["tokens"]],
                                         [int(w) for w in item.get("want", [])]))
            logits = self.runner.step(entries) if entries else None
        except Exception:
            for rid in admitted:
                manager.release(self.live.pop(rid))
            raise
        result = None
        if logits is not None:
            result = logits.to(torch.float32).cpu().numpy().astype("<f4", copy=False)
            if self.out_dir is not None:
                result.tofile(self.out_dir / f"{record['step']}.f32")
        for rid in record.get("end", []):
            request = self.live.pop(str(rid), None)
            if request is not None:
                manager.release(request)
        return result


def replay_stream(replayer: TraceReplayer, lines: Iterable[str], out: IO[str] = sys.stdout) -> None:
    for line in lines:
        line = line.strip()
        if not line:
            continue
        record = json.loads(line)
        replayer.run_step(record)
        print(f"done {record['step']}", file=out, flush=True)


def main(argv: list[str] | None = None) -> int:
    import argparse

    parser = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    parser.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    parser.add_argument("--dtype", choices=("bfloat16", "float32"), default="bfloat16")
    parser.add_argument("--out", required=True, help="folder that receives <step>.f32")
    parser.add_argument("--max-tokens", type=int, required=True,
                        help="most tokens live requests hold at once (each rounded up to 64)")
    parser.add_argument("--page-size", type=int, default=16)
    parser.add_argument("--max-requests", type=int, default=DEFAULT_LIVE_REQUESTS, help="most requests live at a time")
    parser.add_argument("--device", default="cuda:0")
    args = parser.parse_args(argv)
    print("[trace_run] loading model and kernels ...", file=sys.stderr, flush=True)
    # a trace is about arithmetic, not about where the weights came from: any floating storage type is taken
    loaded = load(args.model, device=args.device, dtype=args.dtype, strict_dtype=False)
    replayer = TraceReplayer(loaded, max_tokens=args.max_tokens, page_size=args.page_size, out_dir=args.out,
                             max_requests=args.max_requests)
    replay_stream(replayer, sys.stdin)
    return 0
