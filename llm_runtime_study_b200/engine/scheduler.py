"""Continuous batching above the step function.

What is taken from the reference's ``BatchScheduler`` (mini_llm/generation.py:
112-399): FCFS admission that stops at the first request that does not fit; the
checks of ``add_request``; ``output_limit = min(max_new_tokens, context - prompt)``;
the three finish reasons (an EOS token is emitted, then ``eos``; else the limit:
``context_length`` if the context cut it short, else ``max_new_tokens``); release
of the cache the moment a request finishes; ``abort_all`` on any failure.

What differs: one forward pass per step holds the decoded tokens of the running
requests *and* portions of prompts, cut under a token budget
(``max_tokens_per_step``), where the reference prefills each prompt whole and
alone (mini_llm/generation.py:313-324).  Pages are taken as sequences grow
(``policy="on_demand"``) or for the whole lifetime at admission
(``policy="reserve"``, the reference's rule, mini_llm/generation.py:299-312).

When pages run out (on-demand only): prompt portions are shrunk or left out
first; if the decoded tokens alone still do not fit, the request admitted last
is *preempted*: its pages and slot are given back and it returns to the front of
the queue with its prompt extended by what it has generated, to be recomputed.
Its events are not repeated and its random stream continues where it was.

Two ways of running a step.  With a runner that can draw tokens on the device
(``step_sampled`` / ``decode_sampled``, see ``engine/step.py``) a request's pending
token, position, sampling options and random counter live in its slot record on the
device, and the drawn ids come back through a pinned buffer: the scheduler *launches*
a step and reads its tokens one call later.  While nothing but decoding goes on, the
next decode step is launched before the tokens of the one in flight are read, so the
device never waits for the host; ``step()`` then returns the events of the step
before.  A request that turns out to have ended (an EOS token) has by then been
given one token too many on the device; that token is dropped, and what it wrote
lies in pages and a slot that only later launches on the same stream can reuse.
Whenever anything else is due (an admission, a prompt portion, a preemption) the step in flight is
read first and the host's picture is exact.  With any other runner (the scripted
one of the CPU tests) logits come back to the host and ``sampler.sample`` picks:
the plain path, kept as the oracle of the first.
"""

from __future__ import annotations

import itertools
import time
from collections import deque
from dataclasses import dataclass, field
from typing import Any, Callable, Literal, Sequence

from ..cache.manager import CacheManager, RequestCache
from ..cache.slots import SlotRecord
from ..errors import GenerationError, SamplingError
from ..sampling.config import SamplingConfig
from .step import StepEntry

FinishReason = Literal["eos", "max_new_tokens", "context_length"]


@dataclass(frozen=True, slots=True)
class GenerationEvent:
    """One generated token (mini_llm/generation.py:34-44).  The text fields stay
    empty when no tokenizer is attached."""

    token_id: int | None
    token_index: int | None
    text_delta: str = ""
    text: str = ""
    finish_reason: FinishReason | None = None
    model_seconds: float | None = None
    prompt_token_count: int | None = None


@dataclass
class _Request:
    index: int
    prompt: list[int]               # tokens to (re)compute before decoding continues
    prompt_token_count: int         # of the original prompt
    output_limit: int
    max_new_tokens: int
    sampling: SamplingConfig
    seed: int
    generated: list[int] = field(default_factory=list)
    cache: RequestCache | None = None
    fed: int = 0                    # tokens of ``prompt`` already in the cache
    pending: int | None = None      # sampled token not yet in the cache
    admitted_at: int = 0
    text: str = ""
    finished: bool = False

    @property
    def prefilling(self) -> bool:
        return self.fed < len(self.prompt)


class Scheduler:
    def __init__(
        self, runner: Any, sampler: Any, *, max_batch_size: int, max_seq_len: int,
        eos_token_ids: Sequence[int], vocab_size: int, max_tokens_per_step: int = 2048,
        policy: Literal["on_demand", "reserve"] = "on_demand",
        synchronize: Callable[[], None] | None = None, seed_source: Callable[[], int] | None = None,
        detokenize: Callable[[list[int]], str] | None = None, device_sampling: bool | None = None,
        check_kernels: Callable[[], None] | None = None,
    ) -> None:
        if max_batch_size <= 0:
            raise GenerationError("max_batch_size must be positive")
        if max_tokens_per_step <= 0:
            raise GenerationError("max_tokens_per_step must be positive")
        if max_seq_len <= 0:
            raise GenerationError("max_seq_len must be positive")
        if policy not in ("on_demand", "reserve"):
            raise GenerationError(f"unknown page policy {policy!r}")
        self.runner = runner
        self.manager: CacheManager = runner.manager
        self.sampler = sampler
        self.max_batch_size = max_batch_size
        self.context_limit = max_seq_len
        self.max_tokens_per_step = max_tokens_per_step
        self.policy = policy
        self.vocab_size = vocab_size
        self._eos = frozenset(eos_token_ids)
        self._synchronize = synchronize
        self._seed_source = seed_source
        self._detokenize = detokenize
        self._ids = itertools.count()
        self._admissions = itertools.count()
        self._waiting: deque[_Request] = deque()
        self._running: list[_Request] = []
        self.stats = {"steps": 0, "preemptions": 0, "tokens": 0, "chained_steps": 0}
        # tokens are drawn on the device and read one call later when the runner can do that
        can = hasattr(runner, "decode_sampled") and hasattr(runner, "step_sampled") and hasattr(sampler, "sample_slots")
        self.device_sampling = can if device_sampling is None else bool(device_sampling)
        if self.device_sampling and not can:
            raise GenerationError("this runner or sampler cannot draw tokens on the device")
        self._check_kernels = check_kernels
        self._inflight: tuple[Any, list[_Request], float] | None = None   # (token handle, its requests, launch time)
        self._last_read = 0.0

    # ------------------------------------------------------------- requests
    def add_request(
        self, prompt_token_ids: Sequence[int], *, max_new_tokens: int, sampling: SamplingConfig = SamplingConfig()
    ) -> int:
        """Validate and queue one request; return the index its events carry
        (mini_llm/generation.py:147-191)."""

        if max_new_tokens <= 0:
            raise GenerationError("max_new_tokens must be positive")
        if sampling.top_k is not None and sampling.top_k > self.vocab_size:
            raise SamplingError(f"top_k {sampling.top_k} exceeds vocabulary size {self.vocab_size}")
        prompt = [int(t) for t in prompt_token_ids]
        if not prompt:
            raise GenerationError("a prompt needs at least one token")
        for t in prompt:
            if not 0 <= t < self.vocab_size:
                raise GenerationError(f"token id {t} is outside the vocabulary [0, {self.vocab_size})")
        if len(prompt) > self.context_limit:
            raise GenerationError(
                f"prompt has {len(prompt)} tokens but model context limit is {self.context_limit}"
            )
        output_limit = min(max_new_tokens, self.context_limit - len(prompt))
        required = len(prompt) + output_limit
        if output_limit > 0 and required > self.manager.max_request_tokens:
            raise GenerationError(
                f"request needs {required} cache tokens but the KV cache holds {self.manager.max_request_tokens}"
            )
        seed = sampling.seed
        if seed is None:
            seed = self._seed_source() if self._seed_source else 0
        index = next(self._ids)
        self._waiting.append(_Request(
            index=index, prompt=prompt, prompt_token_count=len(prompt), output_limit=output_limit,
            max_new_tokens=max_new_tokens, sampling=sampling, seed=seed,
        ))
        return index

    @property
    def has_unfinished(self) -> bool:
        return bool(self._waiting or self._running or self._inflight)

    @property
    def num_waiting(self) -> int:
        return len(self._waiting)

    @property
    def num_running(self) -> int:
        return len(self._running)

    def abort_all(self) -> None:
        """Release every running cache and drop every waiting request."""

        running, self._running = self._running, []
        self._waiting.clear()
        self._inflight = None
        for request in running:
            if request.cache is not None:
                self.manager.release(request.cache)

    # ----------------------------------------------------------------- step
    def step(self) -> list[tuple[int, GenerationEvent]]:
        """Advance every running request by one token (or one prompt portion)
        and return the events that are known now: with tokens drawn on the device,
        those of the step launched by the call before.  Any failure aborts every
        request."""

        events: list[tuple[int, GenerationEvent]] = []
        try:
            if self.device_sampling:
                chain = self._chainable()
                if chain:
                    # nothing but decoding: launch the next step, then read the one before
                    started = time.perf_counter()
                    handle = self.runner.decode_sampled([r.cache for r in chain], self.sampler)
                    self._count(len(chain), chained=True)
                    self._read_inflight(events)
                    self._inflight = (handle, chain, started)
                    return events
                self._read_inflight(events)
            plan = self._plan(events)
            # Requests that all wait for pages held by one another make no plan:
            # take the pages of the one admitted last and plan again.
            while not plan and len(self._running) > 1:
                self._preempt_last()
                plan = self._plan(events)
            if plan:
                (self._launch if self.device_sampling else self._run)(plan, events)
            elif self._waiting and not self._running:
                head = self._waiting[0]
                raise GenerationError(
                    f"no progress is possible: nothing is running, and the request at the head of the queue cannot "
                    f"be admitted ({self.manager.free_pages} pages of {self.manager.page_size} tokens and "
                    f"{self.manager.free_slots} request slots are free; it has {len(head.prompt)} prompt tokens). "
                    "Pages or slots are held outside this scheduler."
                )
        except Exception:
            self.abort_all()
            raise
        return events

    def _count(self, tokens: int, chained: bool = False) -> None:
        self.stats["steps"] += 1
        self.stats["tokens"] += tokens
        self.stats["chained_steps"] += chained

    # ------------------------------------------- tokens drawn on the device
    def _chainable(self) -> list[_Request] | None:
        """The requests of the next decode step, if it can be launched before the tokens
        of the step in flight are known: every running request awaits a token of that
        step, nobody can be admitted, and the pages suffice.  A request whose last token
        is the one in flight is left out (it ends whatever that token is); one that ends
        with an EOS token is found out a step late."""

        if self._inflight is None or not self._running:
            return None
        if self._waiting and (self._waiting[0].output_limit == 0
                              or (len(self._running) < self.max_batch_size and self.manager.free_slots)):
            return None
        awaited = {id(r) for r in self._inflight[1]}
        if any(r.prefilling or id(r) not in awaited for r in self._running):
            return None
        going = [r for r in self._running if len(r.generated) + 1 < r.output_limit]
        budget = self.manager.budget()
        if not going or not all(budget.take(self.manager.held(r.cache), r.cache.length + 1) for r in going):
            return None
        return going

    def _read_inflight(self, events: list) -> None:
        """Wait for the step in flight, if any, and turn its tokens into events."""

        if self._inflight is None:
            return
        handle, requests, started = self._inflight
        self._inflight = None
        tokens = handle.tokens()
        now = time.perf_counter()
        seconds = now - max(started, self._last_read)
        self._last_read = now
        for request, token in zip(requests, tokens):
            if not request.finished:        # else: the token after its last, drawn before the end was known
                self._emit(request, int(token), seconds, events)

    def _launch(self, plan: list[tuple[_Request, list[int], bool]], events: list) -> None:
        """Start the planned step with its tokens drawn on the device; do not wait for them."""

        started = time.perf_counter()
        drawing = [r for r, _, wants in plan if wants]
        if not any(r.prefilling for r, _, _ in plan):
            # single decoded tokens only (no request is still feeding its prompt): they are in the slot records already
            handle = self.runner.decode_sampled([r.cache for r in drawing], self.sampler)
        else:
            entries = []
            for request, tokens, wants in plan:
                record = None
                if wants:
                    config = request.sampling
                    record = SlotRecord(position=0, temperature=config.temperature, top_k=config.top_k or 0,
                                        top_p=config.top_p, seed=request.seed, counter=len(request.generated))
                entries.append(StepEntry(request.cache, tokens, [len(tokens) - 1] if wants else [], record))
            handle = self.runner.step_sampled(entries, self.sampler)
        self._count(sum(len(t) for _, t, _ in plan))
        for request, fed_tokens, _ in plan:
            if request.prefilling:
                request.fed += len(fed_tokens)
            request.pending = None
        if handle is not None:
            self._inflight = (handle, drawing, started)

    # ----------------------------------------------------- building a batch
    def _preempt_last(self) -> None:
        victim = max(self._running, key=lambda r: r.admitted_at)
        self._running.remove(victim)
        self.manager.release(victim.cache)
        victim.cache = None
        victim.prompt = victim.prompt[: victim.prompt_token_count] + victim.generated
        victim.fed = 0
        victim.pending = None
        self._waiting.appendleft(victim)
        self.stats["preemptions"] += 1

    def _plan(self, events: list) -> list[tuple[_Request, list[int], bool]]:
        """Decide this step's entries: ``(request, tokens, wants_logits)``."""

        manager = self.manager
        # 1. decoded tokens of running requests: they must fit; preempt if they do not
        while True:
            decoding = [r for r in self._running if not r.prefilling and r.pending is not None]
            budget = manager.budget()
            if all(budget.take(manager.held(r.cache), r.cache.length + 1) for r in decoding) or len(self._running) <= 1:
                break
            self._preempt_last()
        plan: list[tuple[_Request, list[int], bool]] = [(r, [r.pending], True) for r in decoding]
        tokens_left = self.max_tokens_per_step - len(plan)

        def portion_for(request: _Request, cache_length: int, held: list[int]) -> int:
            """Largest portion of the request's remaining prompt that fits the
            token budget and the free pages."""

            remaining = len(request.prompt) - request.fed
            return max(0, min(remaining, tokens_left, budget.room(held) - cache_length))

        # 2. requests already admitted that are still feeding their prompt, oldest first
        for request in sorted((r for r in self._running if r.prefilling), key=lambda r: r.admitted_at):
            if tokens_left <= 0:
                break
            held = manager.held(request.cache)
            n = portion_for(request, request.cache.length, held)
            if n <= 0:
                continue
            budget.take(held, request.cache.length + n)
            tokens_left -= n
            tokens = request.prompt[request.fed : request.fed + n]
            plan.append((request, tokens, request.fed + n == len(request.prompt)))

        # 3. admissions, strictly first come first served
        nothing = [0] * len(manager.groups)
        while self._waiting and tokens_left > 0:
            waiting = self._waiting[0]
            if waiting.output_limit == 0:
                # the prompt fills the context: finish without a slot or a forward pass
                self._waiting.popleft()
                events.append((waiting.index, GenerationEvent(
                    token_id=None, token_index=None, finish_reason="context_length",
                    prompt_token_count=waiting.prompt_token_count)))
                continue
            if len(self._running) >= self.max_batch_size or not manager.free_slots:
                break
            lifetime = waiting.prompt_token_count + waiting.output_limit
            if self.policy == "reserve":
                if not budget.take(nothing, lifetime):
                    break
                n = min(len(waiting.prompt), tokens_left)
            else:
                n = portion_for(waiting, 0, nothing)
                if n <= 0:
                    break
                budget.take(nothing, n)
            self._waiting.popleft()
            waiting.cache = manager.admit()
            waiting.admitted_at = next(self._admissions)
            if self.policy == "reserve":
                manager.grow(waiting.cache, lifetime)
            self._running.append(waiting)
            tokens_left -= n
            plan.append((waiting, waiting.prompt[:n], n == len(waiting.prompt)))
        return plan

    # ------------------------------------------------------- running a batch
    def _run(self, plan: list[tuple[_Request, list[int], bool]], events: list) -> None:
        entries = [StepEntry(r.cache, tokens, [len(tokens) - 1] if wants else []) for r, tokens, wants in plan]
        if self._synchronize:
            self._synchronize()
        started = time.perf_counter()
        logits = self.runner.step(entries)
        sampled_requests = [r for r, _, wants in plan if wants]
        tokens: list[int] = []
        if sampled_requests:
            rows = [(r.sampling, r.seed, len(r.generated)) for r in sampled_requests]
            tokens = self.sampler.sample(logits, rows)
        if self._synchronize:
            self._synchronize()
        seconds = time.perf_counter() - started
        self._count(sum(len(t) for _, t, _ in plan))
        for request, fed_tokens, _ in plan:
            if request.prefilling:
                request.fed += len(fed_tokens)
            request.pending = None
        for request, token in zip(sampled_requests, tokens):
            self._emit(request, int(token), seconds, events)

    def _emit(self, request: _Request, token: int, seconds: float, events: list) -> None:
        request.generated.append(token)
        index = len(request.generated)
        reason: FinishReason | None = None
        if token in self._eos:
            reason = "eos"
        elif index == request.output_limit:
            reason = "context_length" if request.output_limit < request.max_new_tokens else "max_new_tokens"
        delta = ""
        if self._detokenize is not None:
            text = self._detokenize(request.generated)
            if not text.endswith("�"):          # hold back an incomplete UTF-8 sequence
                delta, request.text = text[len(request.text):], text
        events.append((request.index, GenerationEvent(
            token_id=token, token_index=index - 1, text_delta=delta, text=request.text, finish_reason=reason,
            model_seconds=seconds, prompt_token_count=request.prompt_token_count if index == 1 else None)))
        if reason is None:
            request.pending = token
        else:
            request.finished = True
            self.manager.release(request.cache)
            request.cache = None
            self._running.remove(request)
            if self._check_kernels is not None:
                # a kernel whose bounded wait ran out finishes on incomplete data: before this
                # request's tokens count as final, ask whether that ever happened
                self._check_kernels()
