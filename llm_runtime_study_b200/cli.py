"""Command line: ``python -m llm_runtime_study_b200 --model DIR ...``.

Options keep the reference's names and meanings (mini_llm/cli.py:32-64):
``--model --prompt --interactive --max-new-tokens --max-seq-len --temperature
--top-k --top-p --seed --device --dtype --thinking --no-stream --no-metrics``.
Added here: ``--prompt-ids`` (a prompt as token ids, needed when the folder has no
tokenizer), ``--random-weights CONFIG`` with ``--weights-seed`` (write a model
folder with seeded random weights into ``--model`` first), ``--max-batch-size``,
``--page-size``, ``--max-tokens-per-step``, ``--no-cuda-graph``.  Known errors
print ``error: ...`` and exit with 2 (mini_llm/cli.py:273-284).
"""

from __future__ import annotations

import argparse
import json
import sys
import time
from dataclasses import dataclass
from pathlib import Path
from typing import Sequence, TextIO

from .errors import (
    CheckpointError, ConfigError, EngineError, GenerationError, KernelError, KVCacheError, SamplingError,
)
from .sampling import SamplingConfig
from .tokenizer import TokenizerError


@dataclass(frozen=True, slots=True)
class RunMetrics:
    prompt_tokens: int
    generated_tokens: int
    time_to_first_token: float
    decode_seconds: float
    finish_reason: str


def build_parser() -> argparse.ArgumentParser:
    parser = argparse.ArgumentParser(
        prog="python -m llm_runtime_study_b200",
        description="Generate with a Qwen3 dense model on one B200.",
    )
    parser.add_argument("--model", type=Path, required=True)
    parser.add_argument("--prompt", help="raw prompt for one-shot mode, or an optional first interactive prompt")
    parser.add_argument("--prompt-ids", help="prompt as comma- or space-separated token ids")
    parser.add_argument("--interactive", action="store_true", help="load the model once and repeatedly read prompts")
    parser.add_argument("--max-new-tokens", type=int, default=128)
    parser.add_argument("--max-seq-len", type=int, default=4096)
    parser.add_argument("--temperature", type=float, default=0.0)
    parser.add_argument("--top-k", type=int)
    parser.add_argument("--top-p", type=float, default=1.0)
    parser.add_argument("--seed", type=int)
    parser.add_argument("--device", default="auto", help="auto, cuda or cuda:N")
    parser.add_argument("--dtype", choices=("auto", "bfloat16", "float32"), default="auto")
    parser.add_argument("--thinking", action="store_true")
    parser.add_argument("--no-stream", action="store_true")
    parser.add_argument("--no-metrics", action="store_true")
    parser.add_argument("--random-weights", type=Path, metavar="CONFIG",
                        help="config.json to write, with seeded random weights, into --model before loading")
    parser.add_argument("--weights-seed", type=int, default=0)
    parser.add_argument("--max-batch-size", type=int, default=1)
    parser.add_argument("--page-size", type=int, default=16)
    parser.add_argument("--max-tokens-per-step", type=int, default=2048)
    parser.add_argument("--no-cuda-graph", action="store_true")
    return parser


def _sampling_from_args(args: argparse.Namespace) -> SamplingConfig:
    return SamplingConfig(temperature=args.temperature, top_k=args.top_k, top_p=args.top_p, seed=args.seed)


def _engine_from_args(args: argparse.Namespace):
    from .engine.engine import Engine

    if args.random_weights is not None:
        from .weights import write_random_model

        write_random_model(args.model, json.loads(args.random_weights.read_text()), args.weights_seed)
    max_seq_len = args.max_seq_len
    return Engine.from_model_dir(
        args.model, device=args.device, dtype=args.dtype, max_seq_len=max_seq_len,
        max_batch_size=args.max_batch_size, use_cuda_graph=not args.no_cuda_graph,
        page_size=args.page_size, max_tokens_per_step=args.max_tokens_per_step,
    )


def _parse_ids(text: str) -> list[int]:
    try:
        return [int(t) for t in text.replace(",", " ").split()]
    except ValueError as exc:
        raise GenerationError(f"--prompt-ids must be integers: {exc}") from exc


def _run_prompt(engine, prompt, args, *, sampling, output: TextIO, include_load_time: bool = True) -> RunMetrics:
    started = time.perf_counter()
    stream = engine.generate((prompt,), max_new_tokens=args.max_new_tokens, sampling=sampling,
                             enable_thinking=args.thinking)
    events = []
    first_token_at = None
    for _, event in stream:
        if first_token_at is None:
            first_token_at = time.perf_counter()
        events.append(event)
        if not args.no_stream:
            if engine.tokenizer is not None:
                print(event.text_delta, end="", flush=True, file=output)
            elif event.token_id is not None:
                print(event.token_id, end=" ", flush=True, file=output)
    finished = time.perf_counter()
    if not events:
        raise GenerationError("generation ended without a terminal event")
    prompt_tokens = events[0].prompt_token_count
    if prompt_tokens is None:
        raise GenerationError("first generation event is missing prompt-token count")
    if args.no_stream:
        if engine.tokenizer is not None:
            print(events[-1].text, file=output)
        else:
            print(" ".join(str(e.token_id) for e in events if e.token_id is not None), file=output)
    else:
        print(file=output)
    metrics = RunMetrics(
        prompt_tokens=prompt_tokens,
        generated_tokens=sum(e.token_id is not None for e in events),
        time_to_first_token=(first_token_at or finished) - started,
        decode_seconds=sum(e.model_seconds or 0.0 for e in events[1:]),
        finish_reason=events[-1].finish_reason or "unknown",
    )
    if not args.no_metrics:
        _print_metrics(engine, metrics, output=output, include_load_time=include_load_time)
    return metrics


def _print_metrics(engine, metrics: RunMetrics, *, output: TextIO, include_load_time: bool = True) -> None:
    cache_text = "not allocated"
    if engine.last_cache_capacity:
        cache_text = f"{engine.last_cache_num_bytes / (1024**2):.2f} MiB ({engine.last_cache_capacity} positions)"
    decoded = max(0, metrics.generated_tokens - 1)
    rate = decoded / metrics.decode_seconds if decoded and metrics.decode_seconds > 0 else None
    print("\nmetrics", file=output)
    print(f"  device:              {engine.device}", file=output)
    print(f"  dtype:               {engine.dtype}", file=output)
    if include_load_time:
        print(f"  load time:           {engine.load_seconds:.2f} s", file=output)
    print(f"  prompt tokens:       {metrics.prompt_tokens}", file=output)
    print(f"  generated tokens:    {metrics.generated_tokens}", file=output)
    print(f"  cache:               {cache_text}", file=output)
    print(f"  time to first token: {metrics.time_to_first_token * 1_000:.2f} ms", file=output)
    print(f"  decode throughput:   {'n/a' if rate is None else f'{rate:.2f} tokens/s'}", file=output)
    print(f"  stop reason:         {metrics.finish_reason}", file=output)


def run(args: argparse.Namespace, *, output: TextIO) -> RunMetrics:
    if args.prompt is None and args.prompt_ids is None:
        raise GenerationError("--prompt or --prompt-ids is required unless --interactive is used")
    sampling = _sampling_from_args(args)
    engine = _engine_from_args(args)
    prompt = _parse_ids(args.prompt_ids) if args.prompt_ids is not None else args.prompt
    return _run_prompt(engine, prompt, args, sampling=sampling, output=output)


def run_interactive(args: argparse.Namespace, *, input_stream: TextIO, output: TextIO, error: TextIO) -> None:
    """Load once, then serve prompts until ``/quit``, ``/exit`` or end of input
    (mini_llm/cli.py:161-210).  Without a tokenizer a line is a list of token ids."""

    sampling = _sampling_from_args(args)
    engine = _engine_from_args(args)
    print(f"Loaded model on {engine.device} with {engine.dtype} in {engine.load_seconds:.2f} s.", file=output)
    print("Enter a prompt. Use /quit or /exit to stop.", file=output)
    first = args.prompt if args.prompt is not None else args.prompt_ids
    while True:
        if first is not None:
            line, first = first, None
            print(f"you> {line}", file=output)
        else:
            print("you> ", end="", flush=True, file=output)
            line = input_stream.readline()
            if line == "":
                print(file=output)
                return
            line = line.rstrip("\r\n")
        if line.strip() in {"/quit", "/exit"}:
            return
        if not line.strip():
            continue
        print("assistant> ", end="", flush=True, file=output)
        try:
            prompt = line if engine.tokenizer is not None else _parse_ids(line)
            _run_prompt(engine, prompt, args, sampling=sampling, output=output, include_load_time=False)
        except (GenerationError, KVCacheError) as exc:
            print(file=output)
            print(f"error: {exc}", file=error)


def main(argv: Sequence[str] | None = None, *, input_stream: TextIO | None = None,
         output: TextIO | None = None, error: TextIO | None = None) -> int:
    input_stream = sys.stdin if input_stream is None else input_stream
    output = sys.stdout if output is None else output
    error = sys.stderr if error is None else error
    args = build_parser().parse_args(argv)
    try:
        if args.interactive:
            run_interactive(args, input_stream=input_stream, output=output, error=error)
        else:
            run(args, output=output)
    except KeyboardInterrupt:
        print("\nInterrupted.", file=output)
    except (CheckpointError, ConfigError, EngineError, GenerationError, KVCacheError, SamplingError,
            TokenizerError, KernelError) as exc:
        print(f"error: {exc}", file=error)
        return 2
    return 0
