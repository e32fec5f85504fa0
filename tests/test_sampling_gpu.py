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


@pytest.mark.parametrize("vocab", [503, 151936])
def test_drawing_out_of_slot_records_equals_drawing_out_of_rows_and_writes_back(sampler, vocab):
    """The same kernels with their per-row options taken from the requests' slot records: the same tokens,
    and each record afterwards holds the drawn token and a counter advanced by one; other records and the
    other words of the drawn ones are untouched."""

    from llm_runtime_study_b200.cache.slots import COUNTER, LAST_TOKEN, SLOT_WORDS, SlotRecord, SlotTable

    torch.manual_seed(3)
    options = [dict(), dict(temperature=0.7), dict(temperature=1.1, top_k=7), dict(temperature=0.9, top_p=0.7), dict(),
               dict(temperature=1.0, top_k=30, top_p=0.9)]
    rows = len(options)
    logits = (torch.randn(rows, vocab) * 3).cuda()
    specs = [(cfg(**o), (1 << 40) + 17 * r, 5 + r) for r, o in enumerate(options)]
    want = sampler.sample(logits, specs)
    table = SlotTable(16, torch.device("cuda:0"))
    slots = [9, 2, 15, 0, 7, 4]                                   # rows and slots are in different orders
    for slot, (c, seed, counter) in zip(slots, specs):
        table.note(slot, SlotRecord(position=100 + slot, temperature=c.temperature, top_k=c.top_k or 0, top_p=c.top_p,
                                    seed=seed, counter=counter, last_token=-7))
    table.records.copy_(torch.from_numpy(table.mirror))
    before = table.records.clone()
    out = torch.full((rows,), -1, dtype=torch.int32, device="cuda")
    sampler.sample_slots(logits, table.records, torch.tensor(slots, dtype=torch.int32, device="cuda"), out, filtered=True)
    assert out.tolist() == want
    after = table.records.cpu()
    expect = before.cpu().clone()
    for slot, token, (_, _, counter) in zip(slots, want, specs):
        expect[slot, LAST_TOKEN] = token
        expect[slot, COUNTER] = counter + 1
    assert torch.equal(after, expect) and after.shape == (17, SLOT_WORDS)


def test_slot_records_feed_a_decode_step():
    """``slot_store`` writes records by slot; ``slot_load`` turns the records of a batch's slots into token
    ids, positions and lengths, advances the positions of live records and leaves the padding record alone."""

    from llm_runtime_study_b200.cache.slots import POSITION, SlotRecord, SlotTable
    from llm_runtime_study_b200.ops import slots as slot_ops

    table = SlotTable(6, torch.device("cuda:0"))
    chosen = [4, 1, 3]
    staged = torch.tensor([SlotRecord(position=10 * s, last_token=100 + s, temperature=0.5, counter=s).words() for s in chosen],
                          dtype=torch.int32, device="cuda")
    slot_ops.slot_store(table.records, staged, torch.tensor(chosen, dtype=torch.int32, device="cuda"))
    got = table.records.cpu()
    assert torch.equal(got[chosen], staged.cpu()) and int(got[[0, 2, 5, 6]].abs().sum()) == 0
    batch = torch.tensor([3, table.padding_slot, 4, 1], dtype=torch.int32, device="cuda")
    ids, pos, lens = (torch.full((4,), -9, dtype=torch.int32, device="cuda") for _ in range(3))
    slot_ops.slot_load(table.records, batch, ids, pos, lens)
    assert ids.tolist() == [103, 0, 104, 101] and pos.tolist() == [30, 0, 40, 10] and lens.tolist() == [31, 0, 41, 11]
    after = table.records.cpu()
    assert after[:, POSITION].tolist() == [0, 11, 0, 31, 41, 0, 0]
    slot_ops.slot_load(table.records, batch, ids, pos, lens)                    # the next step continues from there
    assert pos.tolist() == [31, 0, 41, 11]
