"""Two layers of real Qwen3-8B size (hidden 4096, 32 query / 8 KV heads of 128, intermediate
12288, vocabulary 151936) with random weights, replayed under the four cuts (whole; the last 32
tokens one by one; portions of changing size down to two tokens; mixed with other requests), in
32-bit and in bfloat16, against the plain implementation.  At these sizes the batches reach the
kernels that tiny models never use: the tcgen05 projections (128 rows and more), the tcgen05
attention (portions of 32 tokens and more), the TMA decode attention, wide weight-streaming
projections, a vocabulary of 151,936.  One request is 2,400 tokens long, so that the prefill
attention runs behind more than 2,048 cached keys and the decode attention over more than 2,048
keys with the number of parts the engine picks for that length.

The plain model runs in float32 on the GPU here (library products with the reduced-precision
matrix mode off; the 2,400-token request would take minutes on the host) and is pinned to the
same plain model on the CPU by one short request."""

import random

import numpy as np
import pytest
import torch

from tests import helpers

pytestmark = pytest.mark.gpu

QWEN3_8B_TWO_LAYERS = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "vocab_size": 151936, "hidden_size": 4096,
    "intermediate_size": 12288, "num_hidden_layers": 2, "num_attention_heads": 32, "num_key_value_heads": 8,
    "head_dim": 128, "max_position_embeddings": 4096, "rms_norm_eps": 1e-6, "rope_theta": 1000000.0,
    "hidden_act": "silu", "attention_bias": False, "tie_word_embeddings": False, "torch_dtype": "bfloat16",
    "bos_token_id": 151643, "eos_token_id": 151645,
}
LENGTHS = [2400, 300, 150, 40]
CHECK_ROWS = 24          # positions per request whose full logit rows are compared
TAIL = 32
# (rms of the differences, largest difference) of a row of logits as fractions of the row's rms: the same
# bounds as for the tiny models (measured here in float32: 6e-6 and 2.7e-5).
TOL = helpers.REPLAY_TOL


def _checked_rows(index: int, length: int) -> list[int]:
    rows = set(random.Random(index).sample(range(length), min(CHECK_ROWS, length))) | {0, length - 1}
    rows |= {p for p in (2047, 2048, 2049, length - TAIL, length - TAIL - 1, length - 2) if 0 <= p < length}
    return sorted(rows)


@pytest.fixture(scope="module")
def material():
    from llm_runtime_study_b200.engine.runtime import load_random

    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False
    # weights are drawn once in bfloat16 so that both runs and the plain model use the same values
    loaded = load_random(QWEN3_8B_TWO_LAYERS, 7, device="cuda:0", dtype="bfloat16", on_device=False)
    on_gpu = {n: t.float().cuda() for n, t in loaded.weights.items()}
    rng = random.Random(5)
    requests = {f"q{i}": helpers.random_tokens(rng, 151936, n) for i, n in enumerate(LENGTHS)}
    rows = {rid: _checked_rows(i, len(t)) for i, (rid, t) in enumerate(requests.items())}
    plain = {"float32": {}, "bfloat16": {}}
    with torch.no_grad():
        for rid, tokens in requests.items():
            plain["float32"][rid] = helpers.plain_logits(on_gpu, QWEN3_8B_TWO_LAYERS, tokens, dtype=torch.float32,
                                                         rows=rows[rid]).double().cpu()
            plain["bfloat16"][rid] = helpers.plain_logits(on_gpu, QWEN3_8B_TWO_LAYERS, tokens, dtype=torch.float32,
                                                          rows=rows[rid], rounded=True).double().cpu()
        # the plain model on the GPU is the plain model on the CPU
        short = list(requests)[-1]
        on_cpu = {n: t.float() for n, t in loaded.weights.items()}
        want = helpers.plain_logits(on_cpu, QWEN3_8B_TWO_LAYERS, requests[short], dtype=torch.float32, rows=rows[short]).double()
        torch.testing.assert_close(plain["float32"][short], want, atol=2e-3 * float(want.abs().max()), rtol=0)
    del on_gpu, on_cpu
    torch.cuda.empty_cache()
    return dict(loaded=loaded, requests=requests, rows=rows, plain=plain)


def _replay(loaded, steps, wanted_rows):
    from llm_runtime_study_b200.engine.replay import TraceReplayer

    # ask for logits only at the checked positions (a row of logits is 600 KB)
    fed = {}
    for record in steps:
        for entry in record["entries"]:
            base = fed.get(entry["id"], 0)
            entry["want"] = [p - base for p in wanted_rows[entry["id"]] if base <= p < base + len(entry["tokens"])]
            fed[entry["id"]] = base + len(entry["tokens"])
    replayer = TraceReplayer(loaded, max_tokens=helpers.pool_tokens(steps), page_size=16)
    outputs = {}
    for record in steps:
        rows = replayer.run_step(record)
        if rows is not None:
            outputs[record["step"]] = torch.from_numpy(np.array(rows))
    replayer.runner.manager.check()
    return helpers.collect_logits(steps, outputs)


def _in_type(loaded, dtype):
    from llm_runtime_study_b200.engine.runtime import LoadedModel
    from llm_runtime_study_b200.models import DecoderModel
    from llm_runtime_study_b200.parts import Runtime

    if dtype == "bfloat16":
        return loaded
    runtime = Runtime(torch.device("cuda:0"), torch.float32)
    model = DecoderModel(loaded.model.description)
    model.load(loaded.weights, runtime)
    return LoadedModel(model, loaded.config, runtime, loaded.weights)


def _drives(requests):
    return {
        "whole": helpers.trace_whole(requests),
        "tail": helpers.trace_decode_tail(requests, tail=TAIL),
        "portions": helpers.trace_chunked(requests, random.Random(8), sizes=(2, 3, 17, 33, 64, 130, 257, 512)),
        "mixed": helpers.trace_mixed(requests, random.Random(3), live_max=3, tail=4, sizes=(2, 17, 33, 64, 130, 400)),
    }


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_real_sizes_under_every_cut(material, dtype):
    loaded = _in_type(material["loaded"], dtype)
    requests, rows = material["requests"], material["rows"]
    drives = _drives(requests)
    assert any(len(e["tokens"]) == 2 for s in drives["portions"] for e in s["entries"])
    assert sum(len(e["tokens"]) == 1 for s in drives["tail"] for e in s["entries"]) >= TAIL * len(requests) - 8
    results = {}
    for name, steps in drives.items():
        got = _replay(loaded, steps, rows)
        results[name] = got
        for rid in requests:
            out = torch.stack([got[rid][p] for p in rows[rid]]).double()
            want = material["plain"][dtype][rid]
            bad, err, top = helpers.first_wrong_row(out, want, TOL[dtype])
            assert bad is None, (
                f"{dtype} {name} request {rid}: first wrong checked position {rows[rid][bad]}, "
                f"rms and largest |diff| / rms {err:.3e}, {top:.3e} (allowed {TOL[dtype]})")
    if dtype == "float32":       # and the bits do not depend on the cut
        for name, other in results.items():
            for rid in requests:
                for p in rows[rid]:
                    assert torch.equal(results["whole"][rid][p], other[rid][p]), (name, rid, p)


def test_captured_decode_has_room_for_the_parts_of_every_length():
    """An engine opened for 32,768 tokens decoding a request of 20,000: the host's choice of parts does not grow
    steadily with the length (21 parts here, 19 at 32,768), and the recorded launch must have room for it.  The
    captured step gives the bits of the same launches issued one by one."""

    from tests.test_generate_gpu import _decode_both_ways
    from llm_runtime_study_b200.engine.runtime import load_random
    from llm_runtime_study_b200.ops import attention_bf16
    from llm_runtime_study_b200.sampling import SamplingConfig

    assert attention_bf16.parts_for(1, 32, 8, 128, 16, 0, 20001) > attention_bf16.parts_for(1, 32, 8, 128, 16, 0, 32768)
    loaded = load_random(dict(QWEN3_8B_TWO_LAYERS, max_position_embeddings=40960), 7, device="cuda:0", dtype="bfloat16",
                         on_device=True)
    rng = random.Random(2)
    for lengths, bound in (((20000,), 32768), ((40, 3000, 9000), 16384)):
        prompts = [helpers.random_tokens(rng, 151936, n) for n in lengths]
        (eager_ids, eager_logits), (graph_ids, graph_logits) = _decode_both_ways(
            loaded, prompts, [list(range(len(prompts)))] * 4, page=16, max_seq_len=bound, sampling=SamplingConfig())
        assert eager_ids == graph_ids
        for a, b in zip(eager_logits, graph_logits):
            assert torch.equal(a, b)


def test_real_sizes_give_the_same_bits_every_time(material):
    """bfloat16 at real sizes, whole prompts (the tcgen05 projections and both prefill attention kernels) and mixed
    steps: three replays, the same bits."""

    requests, rows = material["requests"], material["rows"]
    drives = _drives(requests)
    for name in ("whole", "mixed"):
        first = _replay(material["loaded"], drives[name], rows)
        for _ in range(2):
            again = _replay(material["loaded"], drives[name], rows)
            for rid in requests:
                for p in rows[rid]:
                    assert torch.equal(first[rid][p], again[rid][p]), (name, rid, p)


def test_two_tile_attention_for_portions_of_every_size(material, monkeypatch):
    """The prefill attention with two row tiles per CTA normally serves steps with a portion of 2,048 tokens
    and more (the whole and tail drives above reach it).  Here it serves every step that the tcgen05 attention
    takes at all: portions that fill one row tile or less, an odd number of tiles, tiles that start in the
    middle of a key tile, beside other requests' tokens."""

    from llm_runtime_study_b200.ops import attention_bf16

    monkeypatch.setattr(attention_bf16, "TC_PAIR_MIN_PORTION", attention_bf16.TC_MIN_PORTION)
    requests, rows = material["requests"], material["rows"]
    drives = _drives(requests)
    for name in ("portions", "mixed"):
        got = _replay(material["loaded"], drives[name], rows)
        for rid in requests:
            out = torch.stack([got[rid][p] for p in rows[rid]]).double()
            bad, err, top = helpers.first_wrong_row(out, material["plain"]["bfloat16"][rid], TOL["bfloat16"])
            assert bad is None, (name, rid, rows[rid][bad], err, top)
    attention_bf16.check_tcgen05_error(128)


def test_twelve_rows_decode_through_the_split_k_projections(material):
    """Twelve requests decoded together: 9 to 16 rows send the products with large weights (gate/up, the
    output head) to the tcgen05 split-K kernel instead of the weight-streaming one; the logits still are
    those of the plain model, and those of the same requests decoded six at a time."""

    from llm_runtime_study_b200.engine.replay import TraceReplayer
    from llm_runtime_study_b200.ops import gemm_bf16

    assert gemm_bf16.few_rows_kernel(12, 2 * 12288, 4096) == "splitk" and gemm_bf16.few_rows_kernel(6, 2 * 12288, 4096) == "skinny"
    loaded = material["loaded"]
    rng = random.Random(11)
    requests = {f"d{i}": helpers.random_tokens(rng, 151936, 3 + i % 5) for i in range(12)}
    weights = {n: t.float() for n, t in loaded.weights.items()}
    want = {rid: helpers.plain_logits(weights, QWEN3_8B_TWO_LAYERS, toks, dtype=torch.float32, rows=[len(toks) - 1],
                                      rounded=True)[0].double()
            for rid, toks in requests.items()}

    def last_logits(groups):
        out = {}
        for group in groups:
            replayer = TraceReplayer(loaded, max_tokens=64 * len(group), page_size=16)
            head = {"step": 0, "entries": [{"id": r, "tokens": requests[r][:-1], "want": []} for r in group], "end": []}
            tail = {"step": 1, "entries": [{"id": r, "tokens": requests[r][-1:], "want": [0]} for r in group], "end": list(group)}
            replayer.run_step(head)
            rows = torch.from_numpy(np.array(replayer.run_step(tail)))
            out.update({r: rows[i] for i, r in enumerate(group)})
            replayer.runner.manager.check()
        return out

    ids = list(requests)
    together, by_six = last_logits([ids]), last_logits([ids[:6], ids[6:]])
    for rid in ids:
        for other in (want[rid], by_six[rid].double()):
            bad, err, top = helpers.first_wrong_row(together[rid].double()[None], other[None], TOL["bfloat16"])
            assert bad is None, (rid, err, top)


@pytest.mark.parametrize("dtype,lengths", [("bfloat16", (40, 300, 700)), ("bfloat16", tuple(5 + 17 * i for i in range(12))),
                                           ("float32", (40, 300, 700))])
def test_captured_decode_step_at_real_sizes(material, dtype, lengths):
    """The decode step as generation runs it at head size 128: slot records in, drawn tokens out,
    replayed from a CUDA graph.  Three requests fill a bucket of four with one padded row; twelve go
    to a bucket of sixteen, where the large projections take the split-K kernels.  The engine is
    opened for 4,096 tokens while the requests hold far fewer, so the captured launch (a grid
    sized for 4,096 tokens, told at every replay how many of its parts to use) differs from the eager one
    (sized for the live lengths).  Eight steps, against
    the same launches issued one by one (the same bits in 32-bit) and against the plain model."""

    from tests.test_generate_gpu import _decode_both_ways
    from llm_runtime_study_b200.sampling import SamplingConfig

    loaded = _in_type(material["loaded"], dtype)
    rng = random.Random(len(lengths))
    prompts = [helpers.random_tokens(rng, 151936, n) for n in lengths]
    live = [list(range(len(prompts)))] * 8
    (eager_ids, eager_logits), (graph_ids, graph_logits) = _decode_both_ways(
        loaded, prompts, live, page=16, max_seq_len=4096, sampling=SamplingConfig())
    on_gpu = {n: t.float().cuda() for n, t in material["loaded"].weights.items()}
    sequences = [list(p) for p in prompts]
    for step, (a, b, ia, ib) in enumerate(zip(eager_logits, graph_logits, eager_ids, graph_ids)):
        if dtype == "float32":
            assert torch.equal(a, b), step
        rms = a.double().pow(2).mean(dim=1, keepdim=True).sqrt()
        bad, err, top = helpers.first_wrong_row(b.double().cpu(), a.double().cpu(), TOL[dtype])
        assert bad is None, (step, err, top)
        # against the plain model on everything fed so far (the last step only: a whole forward pass per request)
        if step == len(eager_logits) - 1:
            for row, tokens in enumerate(sequences):
                want = helpers.plain_logits(on_gpu, QWEN3_8B_TWO_LAYERS, tokens, dtype=torch.float32, rows=[len(tokens) - 1],
                                            rounded=dtype == "bfloat16")[0].double().cpu()
                bad, err, top = helpers.first_wrong_row(b[row].double().cpu()[None], want[None], TOL[dtype])
                assert bad is None, (row, err, top)
        top = torch.topk(a, 2, dim=1).values
        for row in range(len(prompts)):
            if ia[row] != ib[row]:      # only a near-tie may be drawn differently; the sequences then part
                assert float(top[row, 0] - top[row, 1]) <= 2 * TOL[dtype][1] * float(rms[row]), (step, row)
                return
            sequences[row].append(ib[row])


def test_a_real_size_folder_through_the_command_line(tmp_path):
    """A model folder of Qwen3-8B width (four layers, two shards, 4 GB) written by the random-weights mode, loaded
    by the command line in a process of its own, and the same folder replayed step by step: the same greedy tokens.
    The loader maps one tensor at a time: the host memory the load adds stays below twice the largest tensor."""

    import json
    import os
    import subprocess
    import sys
    from pathlib import Path

    from llm_runtime_study_b200.engine.replay import TraceReplayer
    from llm_runtime_study_b200.engine.runtime import load
    from llm_runtime_study_b200.weights import write_random_model

    folder = tmp_path / "model"
    write_random_model(folder, dict(QWEN3_8B_TWO_LAYERS, num_hidden_layers=4), 3, shards=2)
    assert (folder / "model.safetensors.index.json").is_file()
    prompt = helpers.random_tokens(random.Random(2), 151936, 40)
    root = Path(__file__).resolve().parent.parent
    done = subprocess.run(
        [sys.executable, "-m", "llm_runtime_study_b200", "--model", str(folder), "--prompt-ids", " ".join(map(str, prompt)),
         "--max-new-tokens", "6", "--max-seq-len", "256", "--no-stream"],
        capture_output=True, text=True, timeout=600, cwd=root, env={**os.environ, "PYTHONDONTWRITEBYTECODE": "1"})
    assert done.returncode == 0, done.stderr[-2000:]
    lines = done.stdout.splitlines()
    generated = [int(t) for t in lines[0].split()]
    assert len(generated) == 6 and "stop reason:         max_new_tokens" in done.stdout
    host_mib = float(next(l for l in lines if "load host memory:" in l).split()[-2])
    largest_mib = 151936 * 4096 * 2 / 2**20
    assert host_mib < 2 * largest_mib, f"loading added {host_mib:.0f} MiB of host memory; the largest tensor is {largest_mib:.0f} MiB"
    # the same folder, replayed: feed the prompt, then the command line's tokens one by one; each must be the argmax
    loaded = load(folder, device="cuda:0", dtype="bfloat16")
    replayer = TraceReplayer(loaded, max_tokens=64, page_size=16)
    rows = replayer.run_step({"step": 0, "entries": [{"id": "a", "tokens": prompt, "want": [len(prompt) - 1]}], "end": []})
    for i, token in enumerate(generated):
        top = torch.topk(torch.from_numpy(np.array(rows[0])), 2)
        assert int(top.indices[0]) == token or float(top.values[0] - top.values[1]) < 5e-2, (i, token, top)
        rows = replayer.run_step({"step": i + 1, "entries": [{"id": "a", "tokens": [token], "want": [0]}], "end": []})
