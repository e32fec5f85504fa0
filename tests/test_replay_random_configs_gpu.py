"""Replay under random configurations: head sizes in steps of 16, any number of
heads and groups, widths and vocabularies that are no power of two, with and
without biases and a tied head.  Each configuration is replayed whole, in
portions and mixed, in both types, against the plain implementation."""

import random

import numpy as np
import pytest
import torch

from tests import helpers

pytestmark = pytest.mark.gpu

TOL = helpers.REPLAY_TOL


def _configuration(case: int):
    rng = random.Random(case)
    kv = rng.choice([1, 2, 3, 4, 8])
    raw = dict(
        helpers.TINY_A,
        head_dim=rng.choice([16, 32, 48, 64, 64, 80, 96, 112, 128, 128, 160, 256]),
        num_key_value_heads=kv,
        num_attention_heads=kv * rng.choice([1, 2, 3, 4, 5, 7, 8]),
        hidden_size=rng.choice([64, 72, 100, 136, 200, 256, 264, 520, 1000, 1024]),
        intermediate_size=rng.choice([96, 104, 130, 272, 500, 768, 1368]),
        vocab_size=rng.choice([97, 256, 503, 1000, 2049, 5003]),
        num_hidden_layers=rng.choice([1, 2, 3]),
        max_position_embeddings=1024,
        rms_norm_eps=rng.choice([1e-6, 1e-5, 3e-6]),
        rope_theta=rng.choice([1e4, 5e4, 1e6]),
        attention_bias=rng.random() < 0.3,
        tie_word_embeddings=rng.random() < 0.4,
    )
    lengths = [rng.choice([1, 2, 5, 33, 64, 65, 130, 200, 300, 520]) for _ in range(5)]
    return raw, lengths, rng


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", [2, 3, 8, 11, 12, 26, 27, 33])
def test_random_configuration(case, dtype, tmp_path):
    from llm_runtime_study_b200.engine.replay import TraceReplayer
    from llm_runtime_study_b200.engine.runtime import load

    raw, lengths, rng = _configuration(case)
    path, weights = helpers.make_model_dir(tmp_path / "model", raw, case, torch_dtype=dtype)
    requests = {f"r{i}": helpers.random_tokens(rng, raw["vocab_size"], n) for i, n in enumerate(lengths)}
    plain = {rid: helpers.plain_for(dtype, weights, raw, tokens) for rid, tokens in requests.items()}
    loaded = load(path, device="cuda:0", dtype=dtype)
    traces = {
        "whole": helpers.trace_whole(requests),
        "mixed": helpers.trace_mixed(requests, random.Random(case), sizes=(2, 3, 8, 40, 130, 260)),
        "portions": helpers.trace_chunked(requests, random.Random(case), sizes=(2, 17, 64, 128, 129, 250)),
    }
    for kind, steps in traces.items():
        replayer = TraceReplayer(loaded, max_tokens=helpers.pool_tokens(steps))
        outputs = {}
        for record in steps:
            rows = replayer.run_step(record)
            if rows is not None:
                outputs[record["step"]] = torch.from_numpy(np.array(rows))
        replayer.runner.manager.check()
        got = helpers.collect_logits(steps, outputs)
        for rid, tokens in requests.items():
            rows = torch.stack([got[rid][p] for p in range(len(tokens))]).double()
            bad, err, top = helpers.first_wrong_row(rows, plain[rid], TOL[dtype])
            assert bad is None, (
                f"{kind}, request {rid}: first wrong position {bad} of {len(tokens)}, "
                f"rms and largest |diff| / rms {err:.3e}, {top:.3e}; configuration {raw}"
            )


def test_many_heads_long_portions_the_same_bits_every_time(tmp_path):
    """272 query heads in groups of 17 (two slices of a KV head's group in the attention kernels), head size 64, prompts
    of 520 and 300 tokens whole: thousands of attention CTAs started longest first.  This is the shape at which a race in
    the prefill attention first showed; the logits are the plain model's and the same bits in five replays."""

    from llm_runtime_study_b200.engine.replay import TraceReplayer
    from llm_runtime_study_b200.engine.runtime import load

    raw = dict(helpers.TINY_A, vocab_size=1000, hidden_size=72, intermediate_size=98, num_hidden_layers=1,
               num_attention_heads=272, num_key_value_heads=16, head_dim=64, max_position_embeddings=1024,
               rms_norm_eps=1e-5, rope_theta=1e4, attention_bias=True, tie_word_embeddings=False)
    path, weights = helpers.make_model_dir(tmp_path / "model", raw, 3072, torch_dtype="bfloat16")
    rng = random.Random(3072)
    requests = {f"r{i}": helpers.random_tokens(rng, 1000, n) for i, n in enumerate([65, 520, 33, 300])}
    plain = {rid: helpers.plain_for("bfloat16", weights, raw, tokens) for rid, tokens in requests.items()}
    loaded = load(path, device="cuda:0", dtype="bfloat16")
    steps = helpers.trace_whole(requests)
    first = None
    for _ in range(5):
        replayer = TraceReplayer(loaded, max_tokens=helpers.pool_tokens(steps))
        outputs = {r["step"]: torch.from_numpy(np.array(replayer.run_step(r))) for r in steps}
        got = helpers.collect_logits(steps, outputs)
        rows = {rid: torch.stack([got[rid][p] for p in range(len(t))]) for rid, t in requests.items()}
        if first is None:
            first = rows
            for rid in requests:
                bad, err, top = helpers.first_wrong_row(rows[rid].double(), plain[rid], TOL["bfloat16"])
                assert bad is None, (rid, bad, err, top)
        else:
            for rid in requests:
                assert torch.equal(rows[rid], first[rid]), rid
