"""Decode and prefill throughput of the engine at Qwen3-8B shape on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

One JSON line: ``value`` is decoded tokens per second at batch 8 with 2,048
cached tokens per request (device time, CUDA events around K decode steps as
generation runs them: slot records in, drawn tokens out, ids copied to the host);
``e2e`` is the same through the scheduler the Python entry point uses, host token
ids in and out, by the wall clock (batch 1 and 64 under its ``points``); ``prefill`` is one
2,048-token prompt; ``points`` holds decode at batch 1 and 64; ``roofline`` is the
bytes a decode step must read (every weight once plus the live requests' cache)
over its time.  Weights are random (N(0, 0.02); norms 1 + N(0, 0.05)) and token
ids uniform random: there is no network for checkpoints or datasets.  Every
decode step reads far more than the 126 MB L2 holds (16 GB of weights), so no
separate L2 flush is needed between timed iterations.
"""

from __future__ import annotations

import argparse
import gc
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

QWEN3_8B = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "vocab_size": 151936, "hidden_size": 4096,
    "intermediate_size": 12288, "num_hidden_layers": 36, "num_attention_heads": 32, "num_key_value_heads": 8,
    "head_dim": 128, "max_position_embeddings": 4096, "rms_norm_eps": 1e-6, "rope_theta": 1000000.0,
    "hidden_act": "silu", "attention_bias": False, "tie_word_embeddings": False, "torch_dtype": "bfloat16",
    "bos_token_id": 151643, "eos_token_id": 151645,
}
CONTEXT = 2048          # cached tokens per request when decoding
PREFILL_TOKENS = 2048
PAGE_SIZE = 16


def peaks() -> dict:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            raw = json.load(open(path))
            return {"hbm_gbs": float(raw["hbm_gbs"]), "bf16_tflops": float(raw["bf16_tflops"]),
                    "bf16_tflops_sustained": float(raw.get("bf16_tflops_sustained", raw["bf16_tflops"])),
                    "source": "measured"}
        except Exception:
            pass
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed
    region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int = 0) -> None:
        self.lines: list[str] = []
        self.process = None
        try:
            self.process = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100", "-i", str(index)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.process = None

    def _read(self) -> None:
        for line in self.process.stdout:
            self.lines.append(line.strip())

    def mark(self) -> int:
        return len(self.lines)

    def stop(self, start: int = 0) -> dict:
        if self.process is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.process.terminate()
        rows = [l.split(", ") for l in self.lines[start:] if l.count(",") >= 7] or [l.split(", ") for l in self.lines if l.count(",") >= 7]
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in rows for n, v in zip(names, r[4:8]) if v.strip().lower() == "active"})
        mhz = [float(r[0]) for r in rows]
        return {"sm_mhz": statistics.median(mhz), "sm_max_mhz": float(rows[0][1]), "reasons": reasons,
                "power_w": statistics.median(float(r[2]) for r in rows), "samples": len(rows)}


def model_bytes(cfg: dict, layers: int) -> int:
    h, i, v = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    q, kv = cfg["num_attention_heads"] * cfg["head_dim"], cfg["num_key_value_heads"] * cfg["head_dim"]
    per_layer = (q + 2 * kv) * h + h * q + 3 * h * i + 2 * h + 2 * cfg["head_dim"]
    # a decode step reads every layer, the final norm, the head, and one embedding row per token
    return 2 * (layers * per_layer + h + v * h)


def kv_bytes_per_token(cfg: dict, layers: int) -> int:
    return layers * 2 * cfg["num_key_value_heads"] * cfg["head_dim"] * 2


def prefill_flops(cfg: dict, layers: int, tokens: int) -> float:
    h, i, v = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    q, kv = cfg["num_attention_heads"] * cfg["head_dim"], cfg["num_key_value_heads"] * cfg["head_dim"]
    gemm = 2.0 * tokens * layers * ((q + 2 * kv) * h + h * q + 3 * h * i)
    attention = 4.0 * layers * cfg["num_attention_heads"] * cfg["head_dim"] * tokens * (tokens + 1) / 2
    return gemm + attention + 2.0 * v * h


def run_ours(args) -> dict:
    import torch

    from llm_runtime_study_b200.cache.slots import SlotRecord
    from llm_runtime_study_b200.engine.engine import Engine
    from llm_runtime_study_b200.engine.step import StepEntry
    from llm_runtime_study_b200.ops import native

    cfg = dict(QWEN3_8B)
    full_layers = cfg["num_hidden_layers"]
    layers = args.layers or full_layers
    cfg["num_hidden_layers"] = layers
    torch.cuda.set_device(0)
    generator = torch.Generator().manual_seed(0)

    def ids(n):
        return torch.randint(0, cfg["vocab_size"], (n,), generator=generator).tolist()

    max_batch = max(args.batch, 64)
    context = CONTEXT
    if args.only == "decode" and args.context:     # profiling aid: another context length, its own pool size
        context, max_batch = args.context, args.batch
        cfg["max_position_embeddings"] = max(cfg["max_position_embeddings"], context + 1024)
    engine = Engine.from_random_weights(
        cfg, seed=0, device="cuda:0", dtype="bfloat16", max_seq_len=cfg["max_position_embeddings"],
        max_batch_size=max_batch, page_size=PAGE_SIZE,
        max_cache_tokens=max_batch * (context + args.steps + max_batch + max(args.warmup, 3) + 2 * PAGE_SIZE),
        max_tokens_per_step=PREFILL_TOKENS, use_cuda_graph=True)
    runner, manager = engine.runner, engine.cache_manager
    sampler = engine._sampler
    greedy = SlotRecord(position=0)          # temperature 0: the largest logit

    def timed(fn, repeat):
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        for _ in range(repeat):
            fn()
        end.record()
        torch.cuda.synchronize()
        return start.elapsed_time(end) / repeat

    # ------------------------------------------------------------- prefill
    def one_prefill():
        request = manager.admit()
        handle = runner.step_sampled([StepEntry(request, prompt, [PREFILL_TOKENS - 1], greedy)], sampler)
        handle.tokens()
        manager.release(request)

    prompt = ids(PREFILL_TOKENS)
    if args.only == "prefill":  # profiling aid: nothing but prefills of one prompt
        for _ in range(max(args.warmup, 1)):
            one_prefill()
        return {"only": "prefill", "layers": layers, "ms": round(timed(one_prefill, args.steps), 3)}
    prefill_ms = 0.0
    if args.only != "decode":
        for _ in range(max(args.warmup, 3)):
            one_prefill()
        prefill_ms = statistics.median(timed(one_prefill, 1) for _ in range(5))

    # -------------------------------------------------------------- decode
    def decode_point(batch, steps, warmup, sample_clocks=False):
        """The decode step as generation runs it: slot records in, drawn tokens out, replayed from
        a CUDA graph, the drawn ids copied to pinned host memory after every step."""

        requests = [manager.admit() for _ in range(batch)]
        for request in requests:
            for at in range(0, context, PREFILL_TOKENS):
                n = min(PREFILL_TOKENS, context - at)
                last = at + n == context
                runner.step_sampled([StepEntry(request, ids(n), [n - 1] if last else [], greedy if last else None)], sampler)
        handles = []

        def one_step():
            handles.append(runner.decode_sampled(requests, sampler))

        for _ in range(max(warmup, 3)):
            one_step()
        handles.pop().tokens()
        handles.clear()
        clocks = ClockSampler() if sample_clocks else None
        mark = clocks.mark() if clocks else 0
        before = native.launch_count()
        ms = timed(one_step, steps)
        launches = native.launch_count() - before
        info = clocks.stop(mark) if clocks else None
        handles[-1].tokens()
        for request in requests:
            manager.release(request)
        return ms, launches, info

    if args.only == "decode":   # profiling aid: nothing but the decode steps of one batch size
        ms, launches, _ = decode_point(args.batch, args.steps, args.warmup)
        return {"only": "decode", "layers": layers, "batch": args.batch, "context": context, "ms_per_step": round(ms, 4),
                "gpu_launches": launches}
    ms_b8, launches, clocks = decode_point(args.batch, args.steps, args.warmup, sample_clocks=True)
    ms_b1, _, _ = decode_point(1, args.steps, args.warmup)
    ms_b64, _, _ = decode_point(64, args.steps, args.warmup)

    # ------------------------------------- end to end through the scheduler
    def end_to_end(batch):
        """Tokens per second by the wall clock through the scheduler that ``Engine.generate`` drives:
        requests in as host token ids, events with token ids out.  Every step copies its slots and block
        tables from pinned host memory to the device and the drawn ids back into pinned host memory."""

        engine.max_batch_size = batch
        scheduler = engine.create_scheduler()
        for _ in range(batch):
            scheduler.add_request(ids(CONTEXT), max_new_tokens=1024)
        while scheduler.num_waiting or any(r.prefilling for r in scheduler._running):
            scheduler.step()
        for _ in range(max(args.warmup, 3)):
            scheduler.step()
        graph = runner._graphs.graph_for(batch) if runner._graphs else None
        if graph is not None:
            graph.always_send = True          # copy the step's inputs every step, changed or not
        gc.collect()                          # a collection of the host's garbage inside a 60 ms region is milliseconds of noise
        gc.disable()
        try:
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            produced = 0
            for _ in range(args.steps):
                produced += len(scheduler.step())
            torch.cuda.synchronize()
            seconds = time.perf_counter() - t0
        finally:
            gc.enable()
        scheduler.abort_all()
        torch.cuda.synchronize()
        return produced / seconds, (graph.sent * 4 if graph else 0), batch * 4

    e2e_b8, h2d, d2h = end_to_end(args.batch)
    e2e_b1, _, _ = end_to_end(1)
    e2e_b64, _, _ = end_to_end(64)

    pk = peaks()
    step_bytes = model_bytes(cfg, layers) + args.batch * CONTEXT * kv_bytes_per_token(cfg, layers)
    achieved = step_bytes / (ms_b8 * 1e-3) / 1e9
    flops = prefill_flops(cfg, layers, PREFILL_TOKENS)
    value = args.batch / (ms_b8 * 1e-3)
    return {
        "metric": "decode tok/s at batch 8 (2,048 cached tokens each), Qwen3-8B shape",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": round(ms_b8, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: random weights, uniform random token ids", "impl": "ours",
        "config": {
            "model": "Qwen3-8B shape", "layers": layers, "layers_full": full_layers, "hidden": cfg["hidden_size"],
            "q_heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
            "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"], "global_batch": args.batch,
            "seq_len": CONTEXT, "context_limit": cfg["max_position_embeddings"], "page_size": PAGE_SIZE,
            "parallelism": "none (1 GPU)", "cuda_graph": True, "sampling": "greedy, inside the captured step",
            "l2": "inputs larger than L2 (16 GB of weights per step)", "peaks": pk["source"],
        },
        "e2e": {"value": round(e2e_b8, 1), "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "points": {"decode_b1": round(e2e_b1, 1), "decode_b64": round(e2e_b64, 1)}},
        "gpu_launches": launches,
        "prefill": {"value": round(PREFILL_TOKENS / (prefill_ms * 1e-3), 1), "tokens": PREFILL_TOKENS,
                    "ms": round(prefill_ms, 3), "frac": round(flops / (prefill_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": {"decode_b1": round(1 / (ms_b1 * 1e-3), 1), "decode_b64": round(64 / (ms_b64 * 1e-3), 1)},
        "clocks": clocks,
    }


class _IdsTokenizer:
    """Stands in for the tokenizer files, which cannot be had offline: a prompt's
    "text" is its token ids separated by spaces.  It implements the reference's
    ``RuntimeTokenizer`` protocol (mini_llm/tokenizer.py:27-41) and is the only
    object on the reference arm that is not the reference's own."""

    def encode(self, text):
        return [int(t) for t in text.split()]

    def decode(self, token_ids, *, skip_special_tokens=False):
        return " ".join(str(t) for t in token_ids)

    def format_chat(self, messages, *, enable_thinking=False):
        return messages[-1].content


QWEN3_14B = {**QWEN3_8B, "hidden_size": 5120, "intermediate_size": 17408, "num_hidden_layers": 40,
             "num_attention_heads": 40, "num_key_value_heads": 8, "max_position_embeddings": 8192}
QWEN3_32B = {**QWEN3_8B, "hidden_size": 5120, "intermediate_size": 25600, "num_hidden_layers": 64,
             "num_attention_heads": 64, "num_key_value_heads": 8, "max_position_embeddings": 4096}


def _reference_model(cfg: dict):
    """The reference's own Qwen3ForCausalLM with random weights on the GPU (N(0, 0.02); norms 1 + N(0, 0.05))."""

    import torch

    from mini_llm.config import Qwen3Config
    from mini_llm.model.qwen import Qwen3ForCausalLM

    config = Qwen3Config.from_dict({**cfg, "attention_dropout": 0.0})
    device = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    with torch.device("meta"):
        model = Qwen3ForCausalLM(config)
    model.to_empty(device=device)
    generator = torch.Generator(device=device).manual_seed(0)
    with torch.no_grad():
        for name, parameter in model.named_parameters():
            values = torch.empty(parameter.shape, dtype=torch.float32, device=device)
            if name.endswith("norm.weight") or "layernorm" in name:
                values.normal_(1.0, 0.05, generator=generator)
            else:
                values.normal_(0.0, 0.02, generator=generator)
            parameter.data = values.to(torch.bfloat16)
            del values
    model.materialize_derived_buffers(device)
    model.eval().requires_grad_(False)
    return model, device


class _Arm:
    """One implementation behind the two larger workloads: how to open an engine for a configuration, how to
    hand its scheduler a prompt of token ids, and how many tokens its cache holds at the moment.  Everything
    else (arrival times, prompts, what is timed) is the same code for both arms."""

    def __init__(self, impl: str, cfg: dict, *, max_seq_len: int, max_batch: int, pool_tokens: int, budget: int) -> None:
        import torch

        self.impl, self.cfg = impl, cfg
        if impl == "ours":
            from llm_runtime_study_b200.engine.engine import Engine

            self.engine = Engine.from_random_weights(
                cfg, seed=0, device="cuda:0", dtype="bfloat16", max_seq_len=max_seq_len, max_batch_size=max_batch,
                page_size=PAGE_SIZE, max_cache_tokens=pool_tokens, max_tokens_per_step=budget, use_cuda_graph=True)
        else:
            sys.path.insert(0, os.path.join(ROOT, "baseline", "_ref"))
            from mini_llm.engine import Engine

            model, device = _reference_model(cfg)
            # the reference sizes its pool itself: max_seq_len x max_batch_size tokens (mini_llm/engine.py:273-282)
            self.engine = Engine(model=model, tokenizer=_IdsTokenizer(), device=device, dtype=torch.bfloat16,
                                 max_seq_len=max_seq_len, load_seconds=0.0, max_batch_size=max_batch)
        self.torch = torch

    def scheduler(self):
        return self.engine.create_scheduler()

    def add(self, scheduler, token_ids, new_tokens: int) -> int:
        if self.impl == "ours":
            return scheduler.add_request(token_ids, max_new_tokens=new_tokens)
        from mini_llm.tokenizer import ChatMessage

        return scheduler.add_request([ChatMessage(role="user", content=" ".join(map(str, token_ids)))], max_new_tokens=new_tokens)

    def cached_tokens(self) -> int:
        manager = self.engine.cache_manager
        return int(manager.used_tokens) if manager is not None else 0

    def prefilling(self, scheduler) -> bool:
        if self.impl == "ours":
            return bool(scheduler.num_waiting or any(r.prefilling for r in scheduler._running))
        return bool(scheduler.num_waiting)

    def synchronize(self) -> None:
        self.torch.cuda.synchronize()

    def warm(self, prompt, sizes: int) -> None:
        """Requests that end one after the other, so that every batch size up to ``sizes`` has run once
        (kernels built and loaded, every decode graph captured)."""

        scheduler = self.scheduler()
        for i in range(sizes):
            self.add(scheduler, prompt, 3 + i)
        while scheduler.has_unfinished:
            scheduler.step()
        self.synchronize()


def _unavailable(reason: str) -> dict:
    return {"impl": "reference", "unavailable": reason}


def run_staggered_14b(args) -> dict:
    """Qwen3-14B shape: 32 requests arriving 50 ms apart, prompt lengths uniform in [128, 4096], 256 new
    tokens each, continuous batching of at most 16 (the reference's staggered benchmark,
    benchmarks/staggered.py:99-130 and doc/batch.md:45-53, at this model size).  Wall-clock figures through
    each implementation's own scheduler; the reference prefills whole prompts, which is its stock path."""

    import random

    import torch

    cfg = dict(QWEN3_14B)
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    layers = cfg["num_hidden_layers"]
    if args.impl == "reference" and not os.path.isdir(os.path.join(ROOT, "baseline", "_ref", "mini_llm")):
        return _unavailable("the reference is not installed under baseline/_ref")
    torch.cuda.set_device(0)
    rng = random.Random(0)
    generator = torch.Generator().manual_seed(0)
    requests, new_tokens, interval, max_batch = 32, 256, 0.050, 16
    prompts = [torch.randint(0, cfg["vocab_size"], (rng.randint(128, 4096),), generator=generator).tolist()
               for _ in range(requests)]
    try:
        arm = _Arm(args.impl, cfg, max_seq_len=8192, max_batch=max_batch, pool_tokens=max_batch * (4096 + new_tokens + PAGE_SIZE),
                   budget=4096)
        arm.warm(prompts[0][:128], max_batch)
        scheduler = arm.scheduler()
        clocks = ClockSampler()
        arm.synchronize()
        start = time.perf_counter()
        arrival, first, done, index_of = {}, {}, {}, {}
        submitted = produced = steps = 0
        bytes_read = 0.0
        weights, per_token = model_bytes(cfg, layers), kv_bytes_per_token(cfg, layers)
        while submitted < requests or scheduler.has_unfinished:
            now = time.perf_counter() - start
            while submitted < requests and now >= submitted * interval:
                index_of[arm.add(scheduler, prompts[submitted], new_tokens)] = submitted
                arrival[submitted] = submitted * interval
                submitted += 1
            if not scheduler.has_unfinished:
                time.sleep(max(0.0, submitted * interval - now))
                continue
            bytes_read += weights + arm.cached_tokens() * per_token      # what this step has to read at least
            steps += 1
            for index, event in scheduler.step():
                stamp = time.perf_counter() - start
                r = index_of[index]
                first.setdefault(r, stamp)
                produced += event.token_id is not None
                if event.finish_reason is not None:
                    done[r] = stamp
        arm.synchronize()
        makespan = time.perf_counter() - start
        clock_info = clocks.stop()
    except Exception as exc:
        if args.impl == "reference":
            return _unavailable(f"{type(exc).__name__}: {exc}".splitlines()[0][:300])
        raise

    def pct(values, q):
        values = sorted(values)
        return values[min(len(values) - 1, int(round(q * (len(values) - 1))))]

    pk = peaks()
    ttft = [first[r] - arrival[r] for r in range(requests)]
    latency = [done[r] - arrival[r] for r in range(requests)]
    achieved = bytes_read / makespan / 1e9
    config = {"model": "Qwen3-14B shape", "layers": layers, "layers_full": 40, "requests": requests,
              "prompt_tokens": "uniform 128..4096", "new_tokens": new_tokens, "arrival_interval_ms": 50,
              "max_batch_size": max_batch, "page_size": PAGE_SIZE, "steps": steps, "peaks": pk["source"]}
    if args.impl == "ours":
        config.update({"max_tokens_per_step": 4096, "preemptions": scheduler.stats["preemptions"]})
    return {
        "metric": "staggered arrivals, continuous batching: output tok/s (Qwen3-14B shape)", "impl": args.impl,
        "value": round(produced / makespan, 1), "unit": "tokens/s", "n_gpus": 1, "higher_is_better": True, "dtype": "bf16",
        "data": "synthetic: random weights, uniform random token ids", "makespan_s": round(makespan, 3),
        "ttft_ms": {"p50": round(pct(ttft, 0.5) * 1e3, 1), "p95": round(pct(ttft, 0.95) * 1e3, 1)},
        "latency_ms": {"p50": round(pct(latency, 0.5) * 1e3, 1), "p95": round(pct(latency, 0.95) * 1e3, 1)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4),
                     "note": "every step's weights plus the cache live at that step, over the makespan (prompt steps are compute-bound)"},
        "clocks": clock_info, "config": config,
    }


def run_decode_32b(args) -> dict:
    """Qwen3-32B shape: decode at batch 1 and 16 after 1,024-token prompts, 128 new tokens, CUDA-graph decode
    step, through each implementation's own scheduler by the wall clock."""

    import torch

    cfg = dict(QWEN3_32B)
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    layers = cfg["num_hidden_layers"]
    if args.impl == "reference" and not os.path.isdir(os.path.join(ROOT, "baseline", "_ref", "mini_llm")):
        return _unavailable("the reference is not installed under baseline/_ref")
    torch.cuda.set_device(0)
    generator = torch.Generator().manual_seed(0)
    pk = peaks()
    out = {}
    try:
        arm = _Arm(args.impl, cfg, max_seq_len=4096, max_batch=16, pool_tokens=16 * (1024 + 128 + 64), budget=2048)
        clocks = ClockSampler()
        for batch in (1, 16):
            scheduler = arm.scheduler()
            for _ in range(batch):
                arm.add(scheduler, torch.randint(0, cfg["vocab_size"], (1024,), generator=generator).tolist(), 129)
            while arm.prefilling(scheduler):
                scheduler.step()
            for _ in range(8):
                scheduler.step()
            arm.synchronize()
            started = time.perf_counter()
            produced, steps = 0, 0
            while scheduler.has_unfinished and steps < 100:
                produced += len(scheduler.step())
                steps += 1
            arm.synchronize()
            seconds = time.perf_counter() - started
            scheduler.abort_all()
            step_bytes = model_bytes(cfg, layers) + batch * 1088 * kv_bytes_per_token(cfg, layers)
            achieved = step_bytes / (seconds / steps) / 1e9
            out[f"decode_b{batch}"] = {"tokens_per_s": round(produced / seconds, 1), "ms_per_step": round(seconds / steps * 1e3, 3),
                                       "hbm_gbs": round(achieved, 1), "hbm_frac": round(achieved / pk["hbm_gbs"], 4)}
        clock_info = clocks.stop()
    except Exception as exc:
        if args.impl == "reference":
            return _unavailable(f"{type(exc).__name__}: {exc}".splitlines()[0][:300])
        raise
    return {"metric": "decode tok/s at batch 1 and 16 (Qwen3-32B shape, 1,024-token prompts, CUDA-graph decode)", "impl": args.impl,
            "value": out["decode_b16"]["tokens_per_s"], "unit": "tokens/s", "n_gpus": 1, "higher_is_better": True, "dtype": "bf16",
            "data": "synthetic: random weights, uniform random token ids", "points": out,
            "roofline": {"bound": "hbm", "achieved": out["decode_b16"]["hbm_gbs"], "peak": pk["hbm_gbs"], "unit": "GB/s",
                         "frac": out["decode_b16"]["hbm_frac"]},
            "clocks": clock_info,
            "config": {"model": "Qwen3-32B shape", "layers": layers, "layers_full": 64, "prompt_tokens": 1024, "new_tokens": 128,
                       "page_size": PAGE_SIZE, "timing": "wall clock through the scheduler", "peaks": pk["source"]}}


def run_reference(args) -> dict:
    """The unmodified reference from baseline/_ref: its own Qwen3ForCausalLM, paged cache,
    CUDA-graph decode and BatchScheduler, driven through Engine.create_scheduler()."""

    ref = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref, "mini_llm")):
        return {"impl": "reference", "unavailable": "the reference is not installed under baseline/_ref"}
    sys.path.insert(0, ref)
    try:
        import torch

        from mini_llm.engine import Engine
        from mini_llm.tokenizer import ChatMessage

        cfg = dict(QWEN3_8B)
        layers = args.layers or cfg["num_hidden_layers"]
        full_layers = cfg["num_hidden_layers"]
        cfg["num_hidden_layers"] = layers
        model, device = _reference_model(cfg)
        host = torch.Generator().manual_seed(0)

        def prompt(n):
            ids = torch.randint(0, cfg["vocab_size"], (n,), generator=host).tolist()
            return [ChatMessage(role="user", content=" ".join(str(t) for t in ids))]

        def engine_for(batch):
            return Engine(model=model, tokenizer=_IdsTokenizer(), device=device, dtype=torch.bfloat16,
                          max_seq_len=cfg["max_position_embeddings"], load_seconds=0.0, max_batch_size=batch)

        def decode_rate(batch, steps, warmup):
            scheduler = engine_for(batch).create_scheduler()
            for _ in range(batch):
                scheduler.add_request(prompt(CONTEXT), max_new_tokens=1024)
            while scheduler.num_waiting:
                scheduler.step()
            for _ in range(max(warmup, 3)):
                scheduler.step()
            torch.cuda.synchronize()
            started = time.perf_counter()
            produced = 0
            for _ in range(steps):
                produced += len(scheduler.step())
            torch.cuda.synchronize()
            seconds = time.perf_counter() - started
            scheduler.abort_all()
            return produced / seconds, seconds / steps * 1e3

        def prefill_ms():
            times = []
            for _ in range(max(args.warmup, 3) + 5):
                scheduler = engine_for(1).create_scheduler()
                scheduler.add_request(prompt(PREFILL_TOKENS), max_new_tokens=1)
                torch.cuda.synchronize()
                started = time.perf_counter()
                scheduler.step()
                torch.cuda.synchronize()
                times.append((time.perf_counter() - started) * 1e3)
                scheduler.abort_all()
            return statistics.median(times[-5:])

        pre = prefill_ms()
        clocks = ClockSampler()
        rate8, ms8 = decode_rate(args.batch, args.steps, args.warmup)
        clock_info = clocks.stop()
        rate1, _ = decode_rate(1, args.steps, args.warmup)
        rate64, _ = decode_rate(64, args.steps, args.warmup)
        pk = peaks()
        step_bytes = model_bytes(cfg, layers) + args.batch * CONTEXT * kv_bytes_per_token(cfg, layers)
        achieved = step_bytes / (ms8 * 1e-3) / 1e9
        flops = prefill_flops(cfg, layers, PREFILL_TOKENS)
        return {
            "metric": "decode tok/s at batch 8 (2,048 cached tokens each), Qwen3-8B shape", "impl": "reference",
            "value": round(rate8, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": round(ms8, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic: random weights, uniform random token ids",
            "config": {"model": "Qwen3-8B shape", "layers": layers, "layers_full": full_layers, "global_batch": args.batch,
                       "seq_len": CONTEXT, "context_limit": cfg["max_position_embeddings"], "page_size": 16,
                       "parallelism": "none (1 GPU)", "cuda_graph": True,
                       "timing": "wall clock around BatchScheduler.step, synchronised", "peaks": pk["source"]},
            "e2e": {"value": round(rate8, 1), "unit": "tokens/s", "h2d_bytes_per_step": args.batch * 8 * 2,
                    "d2h_bytes_per_step": args.batch * 8},
            "gpu_launches": 0,
            "prefill": {"value": round(PREFILL_TOKENS / (pre * 1e-3), 1), "tokens": PREFILL_TOKENS, "ms": round(pre, 3),
                        "frac": round(flops / (pre * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)},
            "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                         "frac": round(achieved / pk["hbm_gbs"], 4)},
            "points": {"decode_b1": round(rate1, 1), "decode_b64": round(rate64, 1)},
            "clocks": clock_info,
        }
    except Exception as exc:  # the reference or one of its dependencies does not run here
        reason = f"{type(exc).__name__}: {exc}".splitlines()[0][:300]
        return {"impl": "reference", "unavailable": reason}


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=128)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--impl", choices=("ours", "reference"), default="ours")
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--context", type=int, default=0, help="with --only decode: cached tokens per request (default 2048)")
    parser.add_argument("--layers", type=int, default=0, help="fewer layers than the configuration has (named in config)")
    parser.add_argument("--workload", choices=("default", "staggered14b", "decode32b"), default="default",
                        help="default: Qwen3-8B decode/prefill; the others are the larger configurations (either --impl)")
    parser.add_argument("--only", choices=("all", "decode", "prefill"), default="all",
                        help="run only the decode steps or only the prefill (for profiler captures of a small case)")
    args = parser.parse_args()
    if args.gpus != 1:
        print(f"bench.py measures one GPU: --gpus {args.gpus} is not supported by this engine (single-GPU tier)")
        return 2
    if args.workload == "staggered14b":
        result = run_staggered_14b(args)
    elif args.workload == "decode32b":
        result = run_decode_32b(args)
    else:
        result = run_reference(args) if args.impl == "reference" else run_ours(args)
    print(json.dumps(result))
    return 0


if __name__ == "__main__":
    sys.exit(main())
