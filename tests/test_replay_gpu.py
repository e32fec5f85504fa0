"""Replay of the same requests under every way of cutting the work, in 32-bit
and in bfloat16, against the plain implementation: whole; most in one step and
the last 32 tokens one by one; portions of changing size; and mixed batches with
so few pages that they are used again."""

import os
import random
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

from tests import helpers

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent
LENGTHS = {"A": [1, 2, 7, 19, 64, 65, 130, 200], "B": [2, 9, 16, 33, 70, 257, 129, 48], "C": [3, 40, 100, 31, 17]}
TOL = helpers.REPLAY_TOL      # (rms, largest) error of a row of logits as fractions of its root mean square


def _requests(name):
    raw, seed, _ = helpers.TINY[name]
    rng = random.Random(seed + 7)
    return {f"r{i}": helpers.random_tokens(rng, raw["vocab_size"], n) for i, n in enumerate(LENGTHS[name])}


@pytest.fixture(scope="module", params=[(n, d) for n in ("A", "B", "C") for d in ("float32", "bfloat16")],
                ids=lambda p: f"{p[0]}-{p[1]}")
def setup(request, tmp_path_factory):
    from llm_runtime_study_b200.engine.runtime import load

    name, dtype = request.param
    raw, seed, page = helpers.TINY[name]
    path, weights = helpers.make_model_dir(tmp_path_factory.mktemp(f"model{name}{dtype}"), raw, seed, torch_dtype=dtype)
    requests = _requests(name)
    plain = {rid: helpers.plain_for(dtype, weights, raw, toks) for rid, toks in requests.items()}
    loaded = load(path, device="cuda:0", dtype=dtype)
    return dict(name=name, dtype=dtype, raw=raw, page=page, path=path, requests=requests, plain=plain, loaded=loaded)


def _replay(setup, steps, max_tokens=None):
    from llm_runtime_study_b200.engine.replay import TraceReplayer

    replayer = TraceReplayer(setup["loaded"], max_tokens=max_tokens or helpers.pool_tokens(steps), page_size=setup["page"])
    outputs = {}
    for record in steps:
        rows = replayer.run_step(record)
        if rows is not None:
            outputs[record["step"]] = torch.from_numpy(np.array(rows))
    manager = replayer.runner.manager
    manager.check()
    assert manager.active_sequences == 0 and all(a.num_free == manager.num_pages for a in manager.allocators)
    return helpers.collect_logits(steps, outputs), manager


def _compare(setup, got):
    worst = 0.0
    for rid, tokens in setup["requests"].items():
        assert sorted(got[rid]) == list(range(len(tokens))), rid
        rows = torch.stack([got[rid][p] for p in range(len(tokens))]).double()
        bad, err, top = helpers.first_wrong_row(rows, setup["plain"][rid], TOL[setup["dtype"]])
        worst = max(worst, err)
        assert bad is None, (
            f"request {rid}: first wrong position {bad} of {len(tokens)} "
            f"(page size {setup['page']}), rms and largest |diff| / rms {err:.3e}, {top:.3e}"
        )
    return worst


def test_whole(setup):
    got, _ = _replay(setup, helpers.trace_whole(setup["requests"]))
    _compare(setup, got)


def test_decode_tail(setup):
    got, _ = _replay(setup, helpers.trace_decode_tail(setup["requests"], tail=32))
    _compare(setup, got)


def test_chunked(setup):
    got, _ = _replay(setup, helpers.trace_chunked(setup["requests"], random.Random(3)))
    _compare(setup, got)


def fed_before(steps, step, rid) -> int:
    """Tokens of request ``rid`` fed in the steps before ``step``."""

    return sum(len(e["tokens"]) for s in steps if s["step"] < step["step"] for e in s["entries"] if e["id"] == rid)


def test_mixed_with_page_reuse(setup):
    steps = helpers.trace_mixed(setup["requests"], random.Random(5))
    assert max(len(s["entries"]) for s in steps) >= 3
    # a single decoded token of one request beside a portion of another, in one step
    assert any(
        any(len(e["tokens"]) == 1 and fed_before(steps, s, e["id"]) > 0 for e in s["entries"])
        and any(len(e["tokens"]) > 1 for e in s["entries"])
        for s in steps
    )
    budget = helpers.pool_tokens(steps)
    assert budget < sum(-(-len(t) // 64) * 64 for t in setup["requests"].values())   # pages must come back
    got, manager = _replay(setup, steps, max_tokens=budget)
    _compare(setup, got)


def test_cutting_does_not_change_float32_bits(setup):
    """In the 32-bit path every sum has an order fixed by the token's own position,
    so the logits are the same bits however the batch was cut."""

    if setup["dtype"] != "float32":
        pytest.skip("bit equality is a property of the 32-bit kernels")
    whole, _ = _replay(setup, helpers.trace_whole(setup["requests"]))
    for steps in (helpers.trace_decode_tail(setup["requests"], 32), helpers.trace_chunked(setup["requests"], random.Random(11)),
                  helpers.trace_mixed(setup["requests"], random.Random(12))):
        other, _ = _replay(setup, steps)
        for rid in whole:
            for p in whole[rid]:
                assert torch.equal(whole[rid][p], other[rid][p]), (rid, p)


def test_a_replay_gives_the_same_bits_every_time(setup):
    """In both types: the same steps three times over give the same bits (nothing depends on which CTA or warp
    came first)."""

    for steps in (helpers.trace_whole(setup["requests"]), helpers.trace_mixed(setup["requests"], random.Random(12))):
        first, _ = _replay(setup, steps)
        for _ in range(2):
            again, _ = _replay(setup, steps)
            for rid in first:
                for p in first[rid]:
                    assert torch.equal(first[rid][p], again[rid][p]), (rid, p)


def test_long_decoding(setup):
    """One token at a time from the first token on, well past several pages."""

    raw = setup["raw"]
    n = min(raw["max_position_embeddings"], 230)
    tokens = helpers.random_tokens(random.Random(21), raw["vocab_size"], n)
    steps = [{"step": i, "entries": [{"id": "x", "tokens": [t], "want": [0]}], "end": ["x"] if i == n - 1 else []}
             for i, t in enumerate(tokens)]
    from llm_runtime_study_b200.engine.replay import TraceReplayer
    from llm_runtime_study_b200.weights import Checkpoint

    weights = Checkpoint.from_model_dir(setup["path"]).get_tensors()
    want = helpers.plain_for(setup["dtype"], weights, raw, tokens)
    replayer = TraceReplayer(setup["loaded"], max_tokens=256, page_size=setup["page"])
    rows = torch.stack([torch.from_numpy(np.array(replayer.run_step(s)))[0] for s in steps]).double()
    bad, err, top = helpers.first_wrong_row(rows, want, TOL[setup["dtype"]])
    assert bad is None, f"first wrong position {bad}, rms and largest |diff| / rms {err:.3e}, {top:.3e}"


def test_trace_run_program(setup, tmp_path):
    """The program itself: stdin protocol, ``done`` lines, files, exit code."""

    requests = dict(list(setup["requests"].items())[:4])
    steps = helpers.trace_mixed(requests, random.Random(9))
    steps.append({"step": len(steps), "entries": [{"id": "quiet", "tokens": [1, 2, 3], "want": []}], "end": ["quiet"]})
    out = tmp_path / "out"
    proc = subprocess.run(
        [sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(setup["path"]), "--dtype", setup["dtype"],
         "--out", str(out), "--max-tokens", str(helpers.pool_tokens(steps)), "--page-size", str(setup["page"])],
        input=helpers.dump_trace(steps), capture_output=True, text=True, timeout=600,
        env={**os.environ, "PYTHONDONTWRITEBYTECODE": "1"},
    )
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert proc.stdout.split() == [w for s in steps for w in ("done", str(s["step"]))]
    assert not (out / f"{steps[-1]['step']}.f32").exists()           # nothing wanted, nothing written
    vocab = setup["raw"]["vocab_size"]
    outputs = {}
    for s in steps[:-1]:
        data = np.fromfile(out / f"{s['step']}.f32", dtype="<f4")
        wanted = sum(len(e["want"]) for e in s["entries"])
        assert data.size == wanted * vocab
        outputs[s["step"]] = torch.from_numpy(data.reshape(wanted, vocab))
    got = helpers.collect_logits(steps[:-1], outputs)
    setup_small = {**setup, "requests": requests}
    _compare(setup_small, got)
