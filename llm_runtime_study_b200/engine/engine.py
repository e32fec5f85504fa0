"""The Python entry point: ``Engine.from_model_dir(...).generate(...)``.

Names and meanings follow the reference's ``Engine`` (mini_llm/engine.py:144-352):
``from_model_dir(model_dir, *, device, dtype, max_seq_len, max_batch_size,
cache_backend, use_cuda_graph)``, ``generate(...)`` yielding
``(request_index, GenerationEvent)``, ``create_scheduler()``, ``cache_manager``,
``last_cache_num_bytes``, ``last_cache_capacity``, ``synchronize()``.  Prompts are
lists of token ids; when the model folder holds a ``tokenizer.json`` a prompt may
also be a string or a list of chat messages.
"""

from __future__ import annotations

import time
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Iterator, Mapping, Sequence

import torch

from ..cache.manager import CacheManager
from ..errors import EngineError, GenerationError
from ..sampling import Sampler, SamplingConfig, fresh_seed
from .runtime import LoadedModel, load, load_random
from .scheduler import GenerationEvent, Scheduler
from .step import StepRunner


@dataclass
class Engine:
    loaded: LoadedModel
    max_seq_len: int
    load_seconds: float = 0.0
    max_batch_size: int = 1
    cache_backend: str = "paged"
    use_cuda_graph: bool = True
    page_size: int = 16
    max_tokens_per_step: int = 2048
    max_cache_tokens: int | None = None
    page_policy: str = "on_demand"
    strict_dtype: bool = True
    device_sampling: bool = True
    tokenizer: Any = None
    source: Any = None   # how the weights were obtained: ("dir", path) or ("random", config, seed, on_device)
    _runner: StepRunner | None = field(default=None, init=False, repr=False)
    _sampler: Sampler | None = field(default=None, init=False, repr=False)

    def __post_init__(self) -> None:
        if self.max_batch_size <= 0:
            raise EngineError("max_batch_size must be positive")
        if self.cache_backend != "paged":
            raise EngineError(f"unsupported cache backend {self.cache_backend!r}; this engine has the 'paged' cache only")
        self.loaded.config.validate_context_length(self.max_seq_len)

    # ------------------------------------------------------------- loading
    @classmethod
    def from_model_dir(
        cls, model_dir: str | Path, *, device: str | torch.device = "auto", dtype: str | torch.dtype = "auto",
        max_seq_len: int = 4096, max_batch_size: int = 1, cache_backend: str = "paged",
        use_cuda_graph: bool = True, **options: Any,
    ) -> "Engine":
        """Load a folder with ``config.json`` and safetensors weights.  Further
        options: ``page_size``, ``max_tokens_per_step``, ``max_cache_tokens``,
        ``page_policy`` ("on_demand" or "reserve"), ``strict_dtype`` (on by default:
        every floating tensor must be stored in config.json's ``torch_dtype``),
        ``device_sampling`` (on by default: tokens are drawn on the device and a
        request's position, pending token and random counter live in its slot record
        there; off: logits come back to the host for every step)."""

        started = time.perf_counter()
        loaded = load(model_dir, device=device, dtype=dtype, strict_dtype=options.get("strict_dtype", True))
        tokenizer = None
        if (Path(model_dir) / "tokenizer.json").is_file():
            from ..tokenizer import load_tokenizer

            tokenizer = load_tokenizer(model_dir)
        engine = cls(loaded=loaded, max_seq_len=max_seq_len, max_batch_size=max_batch_size,
                     cache_backend=cache_backend, use_cuda_graph=use_cuda_graph, tokenizer=tokenizer,
                     source=("dir", Path(model_dir)), **options)
        engine.synchronize()
        engine.load_seconds = time.perf_counter() - started
        return engine

    @classmethod
    def from_random_weights(
        cls, config: Mapping[str, Any], seed: int = 0, *, device="auto", dtype="auto", max_seq_len: int = 4096,
        max_batch_size: int = 1, use_cuda_graph: bool = True, on_device: bool = True, **options: Any,
    ) -> "Engine":
        """A model of the given ``config.json`` object with seeded random weights
        (linear and embedding N(0, 0.02), norm weights 1 + N(0, 0.05))."""

        started = time.perf_counter()
        loaded = load_random(config, seed, device=device, dtype=dtype, on_device=on_device)
        engine = cls(loaded=loaded, max_seq_len=max_seq_len, max_batch_size=max_batch_size,
                     use_cuda_graph=use_cuda_graph, source=("random", dict(config), seed, on_device), **options)
        engine.synchronize()
        engine.load_seconds = time.perf_counter() - started
        return engine

    # ------------------------------------------------------------ properties
    @property
    def device(self) -> torch.device:
        return self.loaded.runtime.device

    @property
    def dtype(self) -> torch.dtype:
        return self.loaded.runtime.dtype

    @property
    def model(self):
        return self.loaded.model

    @property
    def config(self):
        return self.loaded.config

    def _ensure_runner(self) -> StepRunner:
        """The cache pool is made at first use, sized ``max_seq_len * max_batch_size``
        tokens unless ``max_cache_tokens`` says otherwise (mini_llm/engine.py:273-282)."""

        if self._runner is None:
            tokens = self.max_cache_tokens or self.max_seq_len * self.max_batch_size
            tokens = -(-tokens // self.page_size) * self.page_size
            with torch.cuda.device(self.device):
                self._runner = self.loaded.make_runner(
                    max_tokens=tokens, page_size=self.page_size, max_requests=self.max_batch_size,
                    max_seq_len=self.max_seq_len, max_step_tokens=self.max_tokens_per_step,
                )
                self._runner.use_cuda_graph = self.use_cuda_graph
                self._sampler = Sampler(self.device, max_rows=max(self.max_batch_size, 1))
        return self._runner

    @property
    def runner(self) -> StepRunner:
        return self._ensure_runner()

    @property
    def cache_manager(self) -> CacheManager:
        return self._ensure_runner().manager

    @property
    def last_cache_num_bytes(self) -> int:
        allocation = self.cache_manager.last_allocation
        return allocation.num_bytes if allocation is not None else 0

    @property
    def last_cache_capacity(self) -> int:
        allocation = self.cache_manager.last_allocation
        return allocation.capacity if allocation is not None else 0

    def synchronize(self) -> None:
        torch.cuda.synchronize(self.device)

    def allocate_cache(self, capacity: int):
        """A request's hold on the cache with pages for ``capacity`` tokens
        (mini_llm/engine.py:298-299)."""

        manager = self.cache_manager
        request = manager.admit()
        try:
            manager.grow(request, capacity)
        except Exception:
            manager.release(request)
            raise
        return request

    def release_cache(self, cache) -> None:
        self.cache_manager.release(cache)

    def to(self, *, device: str | torch.device | None = None, dtype: str | torch.dtype | None = None) -> "Engine":
        """Place the model on another CUDA device or in the other run type
        (mini_llm/engine.py:304-347).  The reference converts the resident weights in
        place, which loses precision when widening after a downcast; here the weights
        are read (or drawn) again from their source, so ``float32`` after ``bfloat16``
        has the checkpoint's own values.  Captured graphs and the cache pool are dropped."""

        from .runtime import resolve_device, resolve_dtype

        new_device = self.device if device is None else resolve_device(device)
        new_dtype = self.dtype if dtype is None else resolve_dtype(dtype)
        if new_device == self.device and new_dtype == self.dtype:
            return self
        if self._runner is not None and self._runner.manager.active_sequences:
            raise EngineError("cannot move an engine while request caches are active")
        if self.source is None:
            raise EngineError("this engine does not know where its weights came from and cannot be moved")
        if self.source[0] == "dir":
            self.loaded = load(self.source[1], device=new_device, dtype=new_dtype, strict_dtype=self.strict_dtype)
        else:
            _, config, seed, on_device = self.source
            self.loaded = load_random(config, seed, device=new_device, dtype=new_dtype, on_device=on_device)
        self._runner = None
        self._sampler = None
        self.synchronize()
        return self

    # ------------------------------------------------------------ generation
    def create_scheduler(self) -> Scheduler:
        from ..ops import native

        runner = self._ensure_runner()
        description = self.model.description
        return Scheduler(
            runner, self._sampler, max_batch_size=self.max_batch_size, max_seq_len=self.max_seq_len,
            eos_token_ids=description.eos_token_ids, vocab_size=description.vocab_size,
            max_tokens_per_step=self.max_tokens_per_step, policy=self.page_policy,
            synchronize=self.synchronize, seed_source=fresh_seed,
            detokenize=self.tokenizer.decode if self.tokenizer is not None else None,
            device_sampling=self.device_sampling, check_kernels=native.check_kernel_errors,
        )

    def encode_prompt(self, prompt: Any, *, enable_thinking: bool = False) -> list[int]:
        if isinstance(prompt, (list, tuple)) and prompt and all(isinstance(t, int) for t in prompt):
            return list(prompt)
        if self.tokenizer is None:
            raise GenerationError("prompts must be lists of token ids: the model folder has no tokenizer.json")
        return self.tokenizer.encode_prompt(prompt, enable_thinking=enable_thinking)

    def generate(
        self, prompts: Sequence[Any], *, max_new_tokens: int, sampling: SamplingConfig = SamplingConfig(),
        enable_thinking: bool = False,
    ) -> Iterator[tuple[int, GenerationEvent]]:
        """Generate for every prompt; requests beyond ``max_batch_size`` wait for
        a free slot (mini_llm/engine.py:218-240, mini_llm/generation.py:402-450)."""

        if not prompts:
            raise GenerationError("a generation batch must contain at least one request")
        scheduler = self.create_scheduler()
        for prompt in prompts:
            scheduler.add_request(self.encode_prompt(prompt, enable_thinking=enable_thinking),
                                  max_new_tokens=max_new_tokens, sampling=sampling)

        def iterate() -> Iterator[tuple[int, GenerationEvent]]:
            from ..ops import native

            try:
                with torch.cuda.device(self.device):
                    while scheduler.has_unfinished:
                        yield from scheduler.step()
                    native.check_kernel_errors()
            finally:
                scheduler.abort_all()

        return iterate()
