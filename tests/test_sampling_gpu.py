"""The sampling kernel against the plain sampler."""

import pytest
import torch

from tests.plain import sampling_plain as plain

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def sampler():
    from llm_runtime_study_b200.sampling import Sampler

    return Sampler(torch.device("cuda:0"), max_rows=64)


def cfg(**kw):
    from llm_runtime_study_b200.sampling import SamplingConfig

    return SamplingConfig(**kw)


@pytest.mark.parametrize("vocab", [5, 503, 151936])
def test_greedy_is_argmax_lowest_index_on_ties(sampler, vocab):
    torch.manual_seed(0)
    logits = torch.randn(7, vocab)
    logits[3, vocab // 2] = logits[3, vocab - 1] = 50.0          # a tie: the lower index wins
    got = sampler.sample(logits.cuda(), [(cfg(), 0, 0)] * 7)
    want = logits.argmax(dim=-1).tolist()
    want[3] = vocab // 2
    assert got == want


@pytest.mark.parametrize("vocab", [37, 503, 151936])
@pytest.mark.parametrize("opts", [dict(temperature=0.7), dict(temperature=1.3, top_k=5), dict(temperature=1.0, top_p=0.6),
                                  dict(temperature=0.9, top_k=20, top_p=0.8), dict(temperature=2.0, top_k=1)])
def test_matches_the_plain_sampler(sampler, vocab, opts):
    torch.manual_seed(1)
    rows = 6
    logits = torch.randn(rows, vocab) * 2
    specs = [(cfg(**opts), 1234 + r, 3 * r) for r in range(rows)]
    got = sampler.sample(logits.cuda(), specs)
    for r in range(rows):
        want, scores = plain.sample(logits[r], opts["temperature"], opts.get("top_k"), opts.get("top_p", 1.0), 1234 + r, 3 * r)
        keep = plain.kept_mask(logits[r], opts["temperature"], opts.get("top_k"), opts.get("top_p", 1.0))
        assert keep[got[r]], f"row {r}: token {got[r]} is outside the kept set"
        # equal, or a float32-rounding tie between two perturbed scores
        assert got[r] == want or abs(float(scores[got[r]] - scores[want])) < 1e-4


@pytest.mark.parametrize("rows", [3, 20, 40, 64])
def test_large_odd_vocabulary_every_cluster_size(sampler, rows):
    """40,003 entries (rows after the first are not 16-byte aligned) with 3, 20, 40 and 64 rows: clusters
    of eight, four and two CTAs a row and the single CTA."""

    torch.manual_seed(5)
    vocab, opts = 40003, dict(temperature=0.9, top_k=40, top_p=0.7)
    logits = torch.randn(rows, vocab) * 2
    specs = [(cfg(**opts), 77 + r, r) for r in range(rows)]
    got = sampler.sample(logits.cuda(), specs)
    for r in range(0, rows, max(1, rows // 8)):
        want, scores = plain.sample(logits[r], opts["temperature"], opts["top_k"], opts["top_p"], 77 + r, r)
        keep = plain.kept_mask(logits[r], opts["temperature"], opts["top_k"], opts["top_p"])
        assert keep[got[r]], f"row {r}: token {got[r]} is outside the kept set"
        assert got[r] == want or abs(float(scores[got[r]] - scores[want])) < 1e-4


def test_rows_are_independent_of_the_batch(sampler):
    torch.manual_seed(2)
    logits = torch.randn(8, 503).cuda()
    specs = [(cfg(temperature=0.8, top_p=0.9, seed=None), 99, c) for c in range(8)]
    together = sampler.sample(logits, specs)
    alone = [sampler.sample(logits[i : i + 1].contiguous(), [specs[i]])[0] for i in range(8)]
    assert together == alone
    assert len(set(together)) > 1


def test_distribution(sampler):
    logits = torch.tensor([[0.0, 1.0, 2.0, -1.0, 0.5]]).repeat(64, 1).cuda()
    counts = torch.zeros(5)
    for batch in range(40):
        for t in sampler.sample(logits, [(cfg(temperature=1.0), 7, batch * 64 + i) for i in range(64)]):
            counts[t] += 1
    assert float((counts / counts.sum() - torch.softmax(logits[0].cpu(), 0)).abs().max()) < 0.03


def test_non_finite_logits_are_an_error(sampler):
    from llm_runtime_study_b200.errors import SamplingError

    logits = torch.zeros(2, 100)
    logits[1, 5] = float("nan")
    with pytest.raises(SamplingError, match="finite"):
        sampler.sample(logits.cuda(), [(cfg(), 0, 0)] * 2)
    with pytest.raises(SamplingError, match="top_k"):
        sampler.sample(torch.zeros(1, 10).cuda(), [(cfg(temperature=1.0, top_k=11), 0, 0)])
