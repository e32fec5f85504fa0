"""Command line: ``python -m llm_runtime_study_b200 --model DIR ...``.

The options, the metrics block and the exit codes are the reference's
(mini_llm/cli.py:32-64, 213-247, 273-284): ``--model --prompt --interactive
--max-new-tokens --max-seq-len --temperature --top-k --top-p --seed --device --dtype
--thinking --no-stream --no-metrics``; a known error prints ``error: ...`` and exits
with 2.  Added here: ``--prompt-ids`` (the prompt as token ids: the engine proper
starts at token ids, and a folder of random weights has no tokenizer),
``--random-weights CONFIG`` with ``--weights-seed`` (write a model folder with seeded
random weights into ``--model`` first), ``--max-batch-size``, ``--page-size``,
``--max-tokens-per-step``, ``--no-cuda-graph``, ``--any-storage-dtype``.

The program is a thin shell around one ``Session``: it loads an ``Engine`` once, turns
every prompt into token ids, submits it to a scheduler of the engine and consumes that
scheduler's events, printing tokens (or text, when the folder has a tokenizer) as they
arrive and timing what it sees.
"""

from __future__ import annotations

import argparse
import json
import resource
import sys
import time
from pathlib import Path
from typing import Sequence, TextIO

from .errors import (
    CheckpointError, ConfigError, EngineError, GenerationError, KernelError, KVCacheError, SamplingError,
)
from .sampling import SamplingConfig
from .tokenizer import TokenizerError

KNOWN_ERRORS = (CheckpointError, ConfigError, EngineError, GenerationError, KVCacheError, SamplingError,
                TokenizerError, KernelError)
QUIT_WORDS = ("/quit", "/exit")


def build_parser() -> argparse.ArgumentParser:
    parser = argparse.ArgumentParser(
        prog="python -m llm_runtime_study_b200",
        description="Generate with a Qwen3 dense model on one B200.",
    )
    add = parser.add_argument
    add("--model", type=Path, required=True)
    add("--prompt", help="raw prompt for one-shot mode, or an optional first interactive prompt")
    add("--prompt-ids", help="prompt as comma- or space-separated token ids")
    add("--interactive", action="store_true", help="load the model once and repeatedly read prompts")
    add("--max-new-tokens", type=int, default=128)
    add("--max-seq-len", type=int, default=4096)
    add("--temperature", type=float, default=0.0)
    add("--top-k", type=int)
    add("--top-p", type=float, default=1.0)
    add("--seed", type=int)
    add("--device", default="auto", help="auto, cuda or cuda:N")
    add("--dtype", choices=("auto", "bfloat16", "float32"), default="auto")
    add("--thinking", action="store_true")
    add("--no-stream", action="store_true")
    add("--no-metrics", action="store_true")
    add("--random-weights", type=Path, metavar="CONFIG",
        help="config.json to write, with seeded random weights, into --model before loading")
    add("--weights-seed", type=int, default=0)
    add("--max-batch-size", type=int, default=1)
    add("--page-size", type=int, default=16)
    add("--max-tokens-per-step", type=int, default=2048)
    add("--no-cuda-graph", action="store_true")
    add("--any-storage-dtype", action="store_true",
        help="accept weights stored in another floating type than config.json's torch_dtype")
    return parser


def parse_token_ids(text: str) -> list[int]:
    try:
        return [int(word) for word in text.replace(",", " ").split()]
    except ValueError as exc:
        raise GenerationError(f"--prompt-ids must be integers: {exc}") from exc


def _peak_host_mib() -> float:
    return resource.getrusage(resource.RUSAGE_SELF).ru_maxrss / 1024.0


class Completion:
    """What one request produced, and when."""

    def __init__(self) -> None:
        self.token_ids: list[int] = []
        self.text = ""
        self.prompt_tokens: int | None = None
        self.stop_reason: str | None = None
        self.first_token_seconds: float | None = None     # from submission to the first event
        self.decode_seconds = 0.0                         # model time of the steps after the first token


class Session:
    """An engine loaded once and the printing of its completions."""

    def __init__(self, args: argparse.Namespace, output: TextIO) -> None:
        from .engine.engine import Engine

        self.args, self.output = args, output
        self.sampling = SamplingConfig(temperature=args.temperature, top_k=args.top_k, top_p=args.top_p, seed=args.seed)
        if args.random_weights is not None:
            from .weights import write_random_model

            write_random_model(args.model, json.loads(args.random_weights.read_text()), args.weights_seed)
        before = _peak_host_mib()
        self.engine = Engine.from_model_dir(
            args.model, device=args.device, dtype=args.dtype, max_seq_len=args.max_seq_len,
            max_batch_size=args.max_batch_size, use_cuda_graph=not args.no_cuda_graph, page_size=args.page_size,
            max_tokens_per_step=args.max_tokens_per_step, strict_dtype=not args.any_storage_dtype,
        )
        self.load_host_mib = max(0.0, _peak_host_mib() - before)
        self.has_text = self.engine.tokenizer is not None

    def token_ids_of(self, prompt: str, *, is_ids: bool) -> list[int]:
        if is_ids or not self.has_text:
            return parse_token_ids(prompt)
        return self.engine.encode_prompt(prompt, enable_thinking=self.args.thinking)

    def complete(self, prompt_ids: list[int]) -> Completion:
        """Submit one request to a scheduler of the engine and drain its events."""

        done = Completion()
        stream = not self.args.no_stream
        scheduler = self.engine.create_scheduler()
        submitted = time.perf_counter()
        try:
            scheduler.add_request(prompt_ids, max_new_tokens=self.args.max_new_tokens, sampling=self.sampling)
            while scheduler.has_unfinished:
                for _, event in scheduler.step():
                    if done.first_token_seconds is None:
                        done.first_token_seconds = time.perf_counter() - submitted
                        done.prompt_tokens = event.prompt_token_count
                    elif event.model_seconds:
                        done.decode_seconds += event.model_seconds
                    if event.token_id is not None:
                        done.token_ids.append(event.token_id)
                        if stream:
                            piece = event.text_delta if self.has_text else f"{event.token_id} "
                            print(piece, end="", flush=True, file=self.output)
                    done.text = event.text
                    done.stop_reason = event.finish_reason or done.stop_reason
        finally:
            scheduler.abort_all()
        if done.first_token_seconds is None or done.prompt_tokens is None:
            raise GenerationError("generation ended without a terminal event")
        if stream:
            print(file=self.output)
        else:
            print(done.text if self.has_text else " ".join(map(str, done.token_ids)), file=self.output)
        return done

    def report(self, done: Completion, *, with_load: bool) -> None:
        engine, out = self.engine, self.output
        cache = "not allocated"
        if engine.last_cache_capacity:
            cache = f"{engine.last_cache_num_bytes / (1024**2):.2f} MiB ({engine.last_cache_capacity} positions)"
        decoded = max(0, len(done.token_ids) - 1)
        rate = f"{decoded / done.decode_seconds:.2f} tokens/s" if decoded and done.decode_seconds > 0 else "n/a"
        rows = [("device:", engine.device), ("dtype:", engine.dtype)]
        if with_load:
            rows += [("load time:", f"{engine.load_seconds:.2f} s"), ("load host memory:", f"{self.load_host_mib:.0f} MiB")]
        rows += [
            ("prompt tokens:", done.prompt_tokens), ("generated tokens:", len(done.token_ids)), ("cache:", cache),
            ("time to first token:", f"{done.first_token_seconds * 1_000:.2f} ms"), ("decode throughput:", rate),
            ("stop reason:", done.stop_reason or "unknown"),
        ]
        print("\nmetrics", file=out)
        for label, value in rows:
            print(f"  {label:<21}{value}", file=out)

    def answer(self, prompt: str, *, is_ids: bool, with_load: bool) -> Completion:
        done = self.complete(self.token_ids_of(prompt, is_ids=is_ids))
        if not self.args.no_metrics:
            self.report(done, with_load=with_load)
        return done


def converse(session: Session, first: str | None, first_is_ids: bool, *, input_stream: TextIO, output: TextIO,
             error: TextIO) -> None:
    """Serve prompts until ``/quit``, ``/exit`` or the end of the input
    (mini_llm/cli.py:161-210).  Without a tokenizer a line is a list of token ids."""

    engine = session.engine
    print(f"Loaded model on {engine.device} with {engine.dtype} in {engine.load_seconds:.2f} s.", file=output)
    print("Enter a prompt. Use /quit or /exit to stop.", file=output)
    pending = [(first, first_is_ids)] if first is not None else []
    while True:
        if pending:
            line, is_ids = pending.pop()
            print(f"you> {line}", file=output)
        else:
            print("you> ", end="", flush=True, file=output)
            raw = input_stream.readline()
            if not raw:                       # end of input
                print(file=output)
                return
            line, is_ids = raw.rstrip("\r\n"), False
        word = line.strip()
        if word in QUIT_WORDS:
            return
        if not word:
            continue
        print("assistant> ", end="", flush=True, file=output)
        try:
            session.answer(line, is_ids=is_ids, with_load=False)
        except (GenerationError, KVCacheError) as exc:       # a bad prompt does not end the session
            print(file=output)
            print(f"error: {exc}", file=error)


def main(argv: Sequence[str] | None = None, *, input_stream: TextIO | None = None,
         output: TextIO | None = None, error: TextIO | None = None) -> int:
    input_stream = input_stream or sys.stdin
    output = output or sys.stdout
    error = error or sys.stderr
    args = build_parser().parse_args(argv)
    given = args.prompt_ids if args.prompt_ids is not None else args.prompt
    try:
        if given is None and not args.interactive:
            raise GenerationError("--prompt or --prompt-ids is required unless --interactive is used")
        session = Session(args, output)
        if args.interactive:
            converse(session, given, args.prompt_ids is not None, input_stream=input_stream, output=output, error=error)
        else:
            session.answer(given, is_ids=args.prompt_ids is not None, with_load=True)
    except KeyboardInterrupt:
        print("\nInterrupted.", file=output)
    except KNOWN_ERRORS as exc:
        print(f"error: {exc}", file=error)
        return 2
    return 0
