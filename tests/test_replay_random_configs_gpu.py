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
