"""Shared test material: two tiny Qwen3 configurations that differ in every
size and option, model folders with random weights, and trace builders."""

from __future__ import annotations

import json
import random
from pathlib import Path

import torch

from tests.plain import qwen3_plain

# Tiny A: 2 layers, hidden 64, 4 q heads / 2 kv heads, head 16 (q width = hidden),
# tied head, theta 1e4, eps 1e-6, page size 4.
TINY_A = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "vocab_size": 256, "hidden_size": 64, "intermediate_size": 128, "num_hidden_layers": 2,
    "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16,
    "max_position_embeddings": 256, "rms_norm_eps": 1e-6, "rope_theta": 10000.0,
    "hidden_act": "silu", "attention_bias": False, "attention_dropout": 0.0,
    "tie_word_embeddings": True, "torch_dtype": "float32", "bos_token_id": 1, "eos_token_id": 2,
}
# Tiny B: 3 layers, hidden 96, 6 q heads / 1 kv head (MQA), head 32 (q width 192 != hidden),
# intermediate 272 and vocab 503 (no powers of two), untied head, theta 1e6, eps 1e-5, page size 8.
TINY_B = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "vocab_size": 503, "hidden_size": 96, "intermediate_size": 272, "num_hidden_layers": 3,
    "num_attention_heads": 6, "num_key_value_heads": 1, "head_dim": 32,
    "max_position_embeddings": 512, "rms_norm_eps": 1e-5, "rope_theta": 1000000.0,
    "hidden_act": "silu", "attention_bias": False, "attention_dropout": 0.0,
    "tie_word_embeddings": False, "torch_dtype": "float32", "bos_token_id": 0, "eos_token_id": [501, 502],
}
# Tiny C: biases on q/k/v, head 48 (a multiple of 16 that is no power of two), 5 q / 5 kv heads.
TINY_C = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "vocab_size": 131, "hidden_size": 80, "intermediate_size": 112, "num_hidden_layers": 1,
    "num_attention_heads": 5, "num_key_value_heads": 5, "head_dim": 48,
    "max_position_embeddings": 384, "rms_norm_eps": 3e-6, "rope_theta": 50000.0,
    "hidden_act": "silu", "attention_bias": True, "attention_dropout": 0.0,
    "tie_word_embeddings": False, "torch_dtype": "float32", "bos_token_id": 0, "eos_token_id": 1,
}
TINY = {"A": (TINY_A, 0, 4), "B": (TINY_B, 1, 8), "C": (TINY_C, 2, 16)}  # config, seed, page size


def make_model_dir(path: Path, config: dict, seed: int, *, torch_dtype: str | None = None, shards: int = 1):
    """Write a model folder; return (path, {name: CPU tensor as stored})."""

    from llm_runtime_study_b200.weights import Checkpoint, write_random_model

    cfg = dict(config)
    if torch_dtype is not None:
        cfg["torch_dtype"] = torch_dtype
    write_random_model(path, cfg, seed, shards=shards)
    return path, Checkpoint.from_model_dir(path).get_tensors()


def plain_logits(weights: dict, config: dict, token_ids, dtype=torch.float64, *, rows=None, rounded: bool = False) -> torch.Tensor:
    """``rounded``: the plain model keeps its activations as a bfloat16 engine stores them."""

    store = qwen3_plain.round_bfloat16 if rounded else qwen3_plain._keep
    return qwen3_plain.forward(weights, config, token_ids, dtype=dtype, rows=rows, store=store)


# How far a row of logits may be from the plain model's, as fractions of the row's root mean square:
# (the root mean square of the differences, the largest difference).
# float32: the engine in 32-bit against the plain model in 64-bit (32-bit at real sizes): only the order of
# the sums differs; seen: 6e-6 and 2.7e-5.
# bfloat16: the plain model (64-bit arithmetic) rounds its activations to bfloat16 where the engine
# stores them, so what is left is the order of the sums, the rounding of the attention weights, and
# roundings that fall the other way here and there (one bfloat16 step is 2^-8 of a value).  The root
# mean square over a row is a steady figure (a wrong key, position or page moves it by tens of per
# cent); the largest of up to 151,936 differences is a tail value of the same noise and gets more room.
# Seen over all rows these tests compare, tiny models and real sizes alike: rms up to 1.35e-2 (median
# 0.6e-2 to 0.9e-2), largest up to 6.2e-2; the bounds are one and a half times that.
REPLAY_TOL = {"float32": (2e-5, 1e-4), "bfloat16": (2e-2, 1e-1)}


def plain_for(dtype: str, weights: dict, config: dict, token_ids, **kw) -> torch.Tensor:
    """The plain logits an engine of run type ``dtype`` is compared with."""

    return plain_logits(weights, config, token_ids, rounded=dtype == "bfloat16", **kw)


def first_wrong_row(got: torch.Tensor, want: torch.Tensor, tol: tuple[float, float]):
    """(index of the first row that is too far off, or None; the worst rms error / rms; the worst error / rms).
    A NaN anywhere in a row makes it wrong."""

    rms = want.pow(2).mean(dim=1, keepdim=True).sqrt().clamp_min(1e-30)
    diff = (got - want).abs() / rms
    worst, mean = diff.max(dim=1).values, diff.pow(2).mean(dim=1).sqrt()
    bad = (~((mean <= tol[0]) & (worst <= tol[1]))).nonzero()
    return (int(bad[0]) if bad.numel() else None), float(mean.max()), float(worst.max())


def random_tokens(rng: random.Random, vocab: int, length: int) -> list[int]:
    return [rng.randrange(vocab) for _ in range(length)]


# ----------------------------------------------------------------- traces
def trace_whole(requests: dict[str, list[int]]) -> list[dict]:
    """Each request alone and whole: one step holding all its tokens."""

    steps = []
    for step, (rid, tokens) in enumerate(requests.items()):
        steps.append({"step": step, "entries": [{"id": rid, "tokens": tokens, "want": list(range(len(tokens)))}], "end": [rid]})
    return steps


def trace_decode_tail(requests: dict[str, list[int]], tail: int = 32) -> list[dict]:
    """Most of each request in one step, its last ``tail`` tokens one by one."""

    steps, step = [], 0
    for rid, tokens in requests.items():
        head = max(1, len(tokens) - tail)
        steps.append({"step": step, "entries": [{"id": rid, "tokens": tokens[:head], "want": list(range(head))}], "end": []})
        step += 1
        for i in range(head, len(tokens)):
            steps.append({"step": step, "entries": [{"id": rid, "tokens": [tokens[i]], "want": [0]}],
                          "end": [rid] if i == len(tokens) - 1 else []})
            step += 1
        if head == len(tokens):
            steps[-1]["end"] = [rid]
    return steps


def trace_chunked(requests: dict[str, list[int]], rng: random.Random, sizes=(2, 3, 5, 7, 13, 16, 17, 31)) -> list[dict]:
    """Each request in portions of changing size, down to two tokens."""

    steps, step = [], 0
    for rid, tokens in requests.items():
        at = 0
        while at < len(tokens):
            n = min(rng.choice(sizes), len(tokens) - at)
            steps.append({"step": step, "entries": [{"id": rid, "tokens": tokens[at:at + n], "want": list(range(n))}],
                          "end": [rid] if at + n == len(tokens) else []})
            at += n
            step += 1
    return steps


def trace_mixed(requests: dict[str, list[int]], rng: random.Random, *, live_max: int = 4, tail: int = 8,
                sizes=(2, 3, 5, 8, 13)) -> list[dict]:
    """Up to ``live_max`` live requests; portions of some beside single tokens
    of others; a request may sit a step out.  Requests are admitted as others
    end, so pages are used again."""

    waiting = list(requests.items())
    live: dict[str, int] = {}  # id -> tokens fed so far
    steps, step = [], 0
    while waiting or live:
        while waiting and len(live) < live_max:
            rid, _ = waiting.pop(0)
            live[rid] = 0
        entries, ended = [], []
        ids = list(live)
        rng.shuffle(ids)
        for rid in ids:
            tokens = requests[rid]
            at = live[rid]
            if len(ids) > 1 and rng.random() < 0.2:
                continue  # sits this step out
            decode_from = max(1, len(tokens) - tail)
            n = 1 if at >= decode_from else min(rng.choice(sizes), decode_from - at)
            entries.append({"id": rid, "tokens": tokens[at:at + n], "want": list(range(n))})
            live[rid] = at + n
            if live[rid] == len(tokens):
                ended.append(rid)
        if not entries:
            continue
        for rid in ended:
            del live[rid]
        steps.append({"step": step, "entries": entries, "end": ended})
        step += 1
    return steps


def collect_logits(steps: list[dict], outputs: dict[int, "torch.Tensor"]) -> dict[str, dict[int, torch.Tensor]]:
    """Key replayed logits by (request, absolute position)."""

    fed: dict[str, int] = {}
    result: dict[str, dict[int, torch.Tensor]] = {}
    for record in steps:
        rows = outputs.get(record["step"])
        r = 0
        for entry in record["entries"]:
            base = fed.get(entry["id"], 0)
            for w in entry["want"]:
                result.setdefault(entry["id"], {})[base + w] = rows[r]
                r += 1
            fed[entry["id"]] = base + len(entry["tokens"])
    return result


def pool_tokens(steps: list[dict]) -> int:
    """Most tokens live requests hold at any time, each rounded up to 64."""

    held: dict[str, int] = {}
    worst = 0
    for record in steps:
        for entry in record["entries"]:
            held[entry["id"]] = held.get(entry["id"], 0) + len(entry["tokens"])
        worst = max(worst, sum(-(-v // 64) * 64 for v in held.values()))
        for rid in record["end"]:
            held.pop(rid, None)
    return worst


def dump_trace(steps: list[dict]) -> str:
    return "".join(json.dumps(s) + "\n" for s in steps)
