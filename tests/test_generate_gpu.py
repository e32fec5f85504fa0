"""Generation through the Python entry point and the command line, against a
plain loop that recomputes the whole sequence for every token."""

import io
import json
import random

import pytest
import torch

from tests import helpers
from tests.plain import sampling_plain

pytestmark = pytest.mark.gpu


def plain_generate(weights, raw, prompt, n, *, temperature=0.0, top_k=None, top_p=1.0, seed=0, eos=()):
    """Greedy or sampled continuation; returns tokens and, per token, the gap
    between the best and second-best score (a tie is a rounding matter)."""

    tokens, gaps = list(prompt), []
    for counter in range(n):
        logits = helpers.plain_logits(weights, raw, tokens)[-1]
        token, scores = sampling_plain.sample(logits, temperature, top_k, top_p, seed, counter)
        top2 = torch.topk(scores, 2).values
        gaps.append(float(top2[0] - top2[1]))
        tokens.append(token)
        if token in eos:
            break
    return tokens[len(prompt):], gaps


def assert_same_until_a_tie(got, want, gaps, tie):
    for i, (g, w) in enumerate(zip(got, want)):
        if g != w:
            assert gaps[i] < tie, f"token {i}: got {g}, plain {w}, gap {gaps[i]:.3e}"
            return        # after a legitimate tie the sequences differ
    assert len(got) == len(want)


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("B", "float32"), ("A", "bfloat16"), ("B", "bfloat16")])
def test_greedy_generation_matches_plain(tmp_path, name, dtype):
    from llm_runtime_study_b200.engine.engine import Engine

    raw, seed, page = helpers.TINY[name]
    path, weights = helpers.make_model_dir(tmp_path / "m", raw, seed, torch_dtype=dtype)
    eos = raw["eos_token_id"] if isinstance(raw["eos_token_id"], list) else [raw["eos_token_id"]]
    rng = random.Random(3)
    prompts = [helpers.random_tokens(rng, raw["vocab_size"], n) for n in (1, 7, 19, 40, 3)]
    engine = Engine.from_model_dir(path, device="cuda:0", dtype=dtype, max_seq_len=128, max_batch_size=3,
                                   page_size=page, max_tokens_per_step=16)
    out = {}
    for index, event in engine.generate(prompts, max_new_tokens=8):
        out.setdefault(index, []).append(event)
    tie = 1e-5 if dtype == "float32" else 3e-2
    for i, prompt in enumerate(prompts):
        want, gaps = plain_generate(weights, raw, prompt, 8, eos=eos)
        got = [e.token_id for e in out[i]]
        assert_same_until_a_tie(got, want, gaps, tie)
        assert out[i][-1].finish_reason in ("max_new_tokens", "eos")
        assert out[i][0].prompt_token_count == len(prompt)
    manager = engine.cache_manager
    manager.check()
    assert manager.active_sequences == 0 and manager.free_pages == manager.num_pages


def test_seeded_temperature_generation_matches_plain(tmp_path):
    """Tiny B, portions of 13 beside running decodes, temperature 0.7, seed 1234."""

    from llm_runtime_study_b200.engine.engine import Engine
    from llm_runtime_study_b200.sampling import SamplingConfig

    raw, seed, page = helpers.TINY["B"]
    path, weights = helpers.make_model_dir(tmp_path / "m", raw, seed)
    rng = random.Random(4)
    prompts = [helpers.random_tokens(rng, raw["vocab_size"], n) for n in (2, 9, 16, 33, 70)]
    engine = Engine.from_model_dir(path, device="cuda:0", dtype="float32", max_seq_len=128, max_batch_size=4,
                                   page_size=page, max_tokens_per_step=13 + 4)
    sampling = SamplingConfig(temperature=0.7, seed=1234)
    runs = []
    for _ in range(2):
        out = {}
        for index, event in engine.generate(prompts, max_new_tokens=12, sampling=sampling):
            out.setdefault(index, []).append(event.token_id)
        runs.append(out)
    assert runs[0] == runs[1]                                   # same seed, same tokens
    for i, prompt in enumerate(prompts):
        want, gaps = plain_generate(weights, raw, prompt, 12, temperature=0.7, seed=1234, eos=raw["eos_token_id"])
        assert_same_until_a_tie(runs[0][i], want, gaps, 1e-4)


@pytest.mark.parametrize("sampled", [False, True], ids=["greedy", "temperature"])
@pytest.mark.parametrize("policy", ["on_demand", "reserve"])
@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("B", "float32"), ("A", "bfloat16"), ("B", "bfloat16")])
def test_pool_too_small_for_all_requests(tmp_path, name, dtype, policy, sampled):
    """Five requests against a pool that holds about half of what they need together.  Taking pages
    on demand, the request admitted last is preempted when the pages run out and is recomputed
    later; its tokens, greedy or drawn with a seed, are those of the plain loop all the same (the
    seeded stream continues where it was).  Reserving whole lifetimes at admission (the reference's
    rule), nobody is preempted and requests wait instead.  Nothing is left in the pool afterwards."""

    from llm_runtime_study_b200.engine.engine import Engine
    from llm_runtime_study_b200.sampling import SamplingConfig

    raw, seed, page = helpers.TINY[name]
    path, weights = helpers.make_model_dir(tmp_path / "m", raw, seed, torch_dtype=dtype)
    eos = raw["eos_token_id"] if isinstance(raw["eos_token_id"], list) else [raw["eos_token_id"]]
    rng = random.Random(17)
    prompts = [helpers.random_tokens(rng, raw["vocab_size"], n) for n in (9, 20, 14, 30, 5)]
    new_tokens = 24
    engine = Engine.from_model_dir(path, device="cuda:0", dtype=dtype, max_seq_len=128, max_batch_size=4,
                                   page_size=page, max_tokens_per_step=16, max_cache_tokens=96, page_policy=policy)
    sampling = SamplingConfig(temperature=0.7, seed=1234) if sampled else SamplingConfig()
    scheduler = engine.create_scheduler()
    index_of = {scheduler.add_request(p, max_new_tokens=new_tokens, sampling=sampling): i for i, p in enumerate(prompts)}
    out = {i: [] for i in range(len(prompts))}
    while scheduler.has_unfinished:
        for index, event in scheduler.step():
            out[index_of[index]].append(event)
        engine.cache_manager.check()
    if policy == "on_demand":
        assert scheduler.stats["preemptions"] > 0
    else:
        assert scheduler.stats["preemptions"] == 0
    tie = (1e-5 if dtype == "float32" else 3e-2) * (4 if sampled else 1)
    for i, prompt in enumerate(prompts):
        kw = dict(temperature=0.7, seed=1234) if sampled else {}
        want, gaps = plain_generate(weights, raw, prompt, new_tokens, eos=eos, **kw)
        got = [e.token_id for e in out[i]]
        assert [e.token_index for e in out[i]] == list(range(len(got)))         # no event twice, none missing
        assert_same_until_a_tie(got, want, gaps, tie)
        assert out[i][-1].finish_reason in ("max_new_tokens", "eos")
    manager = engine.cache_manager
    manager.check()
    assert manager.active_sequences == 0 and manager.free_pages == manager.num_pages and manager.free_slots == 4


def test_command_line(tmp_path):
    from llm_runtime_study_b200.cli import main

    raw, seed, page = helpers.TINY["A"]
    config_path = tmp_path / "config.json"
    config_path.write_text(json.dumps(raw))
    out, err = io.StringIO(), io.StringIO()
    code = main(["--model", str(tmp_path / "m"), "--random-weights", str(config_path), "--weights-seed", str(seed),
                 "--prompt-ids", "5 17 3", "--max-new-tokens", "6", "--max-seq-len", "64", "--dtype", "float32",
                 "--page-size", str(page), "--no-stream"], output=out, error=err)
    assert code == 0, err.getvalue()
    lines = out.getvalue().splitlines()
    generated = [int(t) for t in lines[0].split()]
    from llm_runtime_study_b200.weights import Checkpoint

    weights = Checkpoint.from_model_dir(tmp_path / "m").get_tensors()
    want, gaps = plain_generate(weights, raw, [5, 17, 3], 6, eos=[raw["eos_token_id"]])
    assert_same_until_a_tie(generated, want, gaps, 1e-5)
    text = out.getvalue()
    assert "prompt tokens:       3" in text and "stop reason:" in text and "decode throughput:" in text
    out, err = io.StringIO(), io.StringIO()
    assert main(["--model", str(tmp_path / "m"), "--prompt-ids", "999999"], output=out, error=err) == 2
    assert err.getvalue().startswith("error: ")
    assert main(["--model", str(tmp_path / "none"), "--prompt-ids", "1"], output=out, error=err) == 2


def _decode_both_ways(loaded, prompts, live_by_step, *, page, max_seq_len, sampling):
    """Prefill the prompts, then decode with tokens drawn on the device, eagerly and from CUDA
    graphs; returns for each way the drawn ids and the logits of every step."""

    from llm_runtime_study_b200.cache.slots import SlotRecord
    from llm_runtime_study_b200.engine.step import StepEntry
    from llm_runtime_study_b200.sampling import Sampler

    results = []
    for use_graph in (False, True):
        runner = loaded.make_runner(max_tokens=len(prompts) * max_seq_len, page_size=page, max_requests=len(prompts),
                                    max_seq_len=max_seq_len)
        runner.use_cuda_graph = use_graph
        sampler = Sampler(loaded.runtime.device, max_rows=len(prompts))
        requests = [runner.manager.admit() for _ in prompts]
        records = [SlotRecord(position=0, temperature=sampling.temperature, top_k=sampling.top_k or 0, top_p=sampling.top_p,
                              seed=sampling.seed or 0, counter=0) for _ in prompts]
        first = runner.step_sampled([StepEntry(r, p, [len(p) - 1], rec) for r, p, rec in zip(requests, prompts, records)], sampler)
        ids, logits = [first.tokens()], [runner.last_logits.clone()]
        for live in live_by_step:
            handle = runner.decode_sampled([requests[i] for i in live], sampler)
            ids.append(handle.tokens())
            logits.append(runner.last_logits.clone())
        assert (runner._graphs is not None) is use_graph
        runner.manager.check()
        results.append((ids, logits))
    return results


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_cuda_graph_decode_equals_eager(tmp_path, dtype):
    """The captured decode step (slot records in, drawn tokens out) gives the same logits and the
    same tokens as the same launches issued one by one, for several batch sizes (one padded up to
    its bucket), ragged lengths, block tables that change, greedy and seeded draws."""

    from llm_runtime_study_b200.engine.runtime import load
    from llm_runtime_study_b200.sampling import SamplingConfig

    raw, seed, page = helpers.TINY["B"]
    path, _ = helpers.make_model_dir(tmp_path / "m", raw, seed, torch_dtype=dtype)
    loaded = load(path, device="cuda:0", dtype=dtype)
    rng = random.Random(6)
    prompts = [helpers.random_tokens(rng, raw["vocab_size"], n) for n in (3, 30, 9, 17)]
    live = [[0, 1, 2, 3]] * 6 + [[0, 1, 2]] * 3 + [[0, 1]] * 3          # 4, then 3 (padded to 4), then 2
    for sampling in (SamplingConfig(), SamplingConfig(temperature=0.8, seed=99), SamplingConfig(temperature=0.8, top_k=20, top_p=0.9, seed=5)):
        (eager_ids, eager_logits), (graph_ids, graph_logits) = _decode_both_ways(
            loaded, prompts, live, page=page, max_seq_len=128, sampling=sampling)
        assert eager_ids == graph_ids
        for a, b in zip(eager_logits, graph_logits):
            assert torch.equal(a, b)


def test_graph_buckets_pad_with_empty_rows(tmp_path):
    from llm_runtime_study_b200.engine.graph import DecodeGraphs

    class Manager:
        max_requests = 48

    class Runner:
        manager = Manager()

    graphs = DecodeGraphs(Runner())
    assert [graphs.bucket(n) for n in (1, 2, 3, 5, 8, 9, 33, 48)] == [1, 2, 4, 8, 8, 16, 48, 48]


def test_engine_to_and_cache_handles(tmp_path):
    from llm_runtime_study_b200.engine.engine import Engine
    from llm_runtime_study_b200.errors import EngineError, KVCacheError

    raw, seed, page = helpers.TINY["A"]
    path, weights = helpers.make_model_dir(tmp_path / "m", raw, seed)
    engine = Engine.from_model_dir(path, device="cuda:0", dtype="bfloat16", max_seq_len=64, max_batch_size=2, page_size=page)
    prompt = [5, 17, 3, 9]
    first = [e.token_id for _, e in engine.generate([prompt], max_new_tokens=4)]
    handle = engine.allocate_cache(10)
    assert engine.last_cache_capacity == 12 and engine.last_cache_num_bytes > 0      # three pages of four
    with pytest.raises(EngineError, match="active"):
        engine.to(dtype="float32")
    engine.release_cache(handle)
    engine.release_cache(handle)
    assert engine.to(dtype="bfloat16") is engine
    engine.to(dtype="float32")
    assert engine.dtype == torch.float32
    want, gaps = plain_generate(weights, raw, prompt, 4, eos=[raw["eos_token_id"]])
    got = [e.token_id for _, e in engine.generate([prompt], max_new_tokens=4)]
    assert_same_until_a_tie(got, want, gaps, 1e-5)
    assert_same_until_a_tie(first, want, gaps, 3e-2)
    with pytest.raises(EngineError):
        engine.to(device="cpu")
    with pytest.raises(KVCacheError):
        engine.allocate_cache(10_000)
