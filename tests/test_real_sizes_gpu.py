"""Two layers of real Qwen3-8B size (hidden 4096, 32 query / 8 KV heads of 128, intermediate
12288, vocabulary 151936) with random weights, replayed whole, with a decoded tail and in mixed
portions, in 32-bit and in bfloat16, against the plain implementation.  At these sizes the
batches reach the kernels that tiny models never use: the tcgen05 projection (128 rows and
more), the tcgen05 attention (portions of 32 tokens and more), wide weight-streaming
projections, a vocabulary of 151,936."""

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
LENGTHS = [300, 150, 40]
CHECK_ROWS = 24          # positions per request whose full logit rows are compared


@pytest.fixture(scope="module")
def material():
    from llm_runtime_study_b200.engine.runtime import load_random

    # weights are drawn once in bfloat16 so that both runs and the plain model use the same values
    loaded = load_random(QWEN3_8B_TWO_LAYERS, 7, device="cuda:0", dtype="bfloat16", on_device=False)
    weights = {n: t.float() for n, t in loaded.weights.items()}
    rng = random.Random(5)
    requests = {f"q{i}": helpers.random_tokens(rng, 151936, n) for i, n in enumerate(LENGTHS)}
    rows = {rid: sorted(set(random.Random(i).sample(range(len(t)), min(CHECK_ROWS, len(t))) + [0, len(t) - 1]))
            for i, (rid, t) in enumerate(requests.items())}
    torch.set_num_threads(max(1, torch.get_num_threads()))
    plain = {}
    for rid, tokens in requests.items():
        # float32 plain model (float64 would need 13 GB for these matrices); same formulas
        hidden_rows = helpers.plain_logits(weights, QWEN3_8B_TWO_LAYERS, tokens, dtype=torch.float32)
        plain[rid] = hidden_rows[rows[rid]].double()
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


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_real_sizes_under_every_cut(material, dtype):
    from llm_runtime_study_b200.engine.runtime import LoadedModel
    from llm_runtime_study_b200.models import DecoderModel
    from llm_runtime_study_b200.parts import Runtime

    loaded = material["loaded"]
    if dtype == "float32":
        runtime = Runtime(torch.device("cuda:0"), torch.float32)
        model = DecoderModel(loaded.model.description)
        model.load(loaded.weights, runtime)
        loaded = LoadedModel(model, loaded.config, runtime, loaded.weights)
    requests, rows = material["requests"], material["rows"]
    # float32 GPU against float32 CPU: both carry summation-order noise over K = 12288
    tol = dict(atol=2e-3, rtol=2e-3) if dtype == "float32" else dict(atol=6e-2, rtol=5e-2)
    results = []
    for steps in (helpers.trace_whole(requests), helpers.trace_decode_tail(requests, tail=6),
                  helpers.trace_mixed(requests, random.Random(3), live_max=3, tail=4, sizes=(2, 17, 33, 64, 130))):
        got = _replay(loaded, steps, rows)
        results.append(got)
        for rid in requests:
            out = torch.stack([got[rid][p] for p in rows[rid]]).double()
            want = material["plain"][rid]
            scale = float(want.abs().max())
            diff = (out - want).abs()
            bad = (diff > tol["atol"] * scale + tol["rtol"] * want.abs()).any(dim=1).nonzero()
            assert bad.numel() == 0, (
                f"{dtype} request {rid}: first wrong checked position {rows[rid][int(bad[0])]}, "
                f"max |diff| {float(diff.max()):.3e} at logit scale {scale:.3f}")
    if dtype == "float32":       # and the bits do not depend on the cut
        for other in results[1:]:
            for rid in requests:
                for p in rows[rid]:
                    assert torch.equal(results[0][rid][p], other[rid][p]), (rid, p)


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
    want = {rid: helpers.plain_logits(weights, QWEN3_8B_TWO_LAYERS, toks, dtype=torch.float32)[-1].double()
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
        scale = float(want[rid].abs().max())
        torch.testing.assert_close(together[rid].double(), want[rid], atol=6e-2 * scale, rtol=5e-2)
        torch.testing.assert_close(together[rid].double(), by_six[rid].double(), atol=3e-2 * scale, rtol=3e-2)
