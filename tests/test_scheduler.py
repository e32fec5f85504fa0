"""The scheduler's decisions, with the real step bookkeeping and cache manager on
the CPU and a scripted model in place of the network (no GPU).  The scripted
model answers "next token = last token + 1", so every output is known."""

import pytest
import torch

from llm_runtime_study_b200.cache import CacheLayout, CacheManager
from llm_runtime_study_b200.engine.scheduler import Scheduler
from llm_runtime_study_b200.engine.step import StepRunner
from llm_runtime_study_b200.errors import GenerationError, KVCacheError, SamplingError
from llm_runtime_study_b200.parts.base import PagedKV, Runtime
from llm_runtime_study_b200.sampling import SamplingConfig

VOCAB, EOS = 50, 49


class ScriptedModel:
    def __init__(self):
        self.batches = []      # [(entry lengths, positions)] as seen by the model
        self.fail_at = None

    def bind_cache(self, manager):
        pass

    def forward(self, ctx):
        if self.fail_at is not None and len(self.batches) == self.fail_at:
            raise RuntimeError("injected failure")
        self.batches.append((list(ctx.q_lens), ctx.positions.tolist(), list(ctx.kv_lens)))
        if ctx.num_logit_rows == 0:
            return None
        last = ctx.token_ids[ctx.logit_rows.long()].long()
        return torch.nn.functional.one_hot((last + 1) % VOCAB, VOCAB).float()


class ArgmaxSampler:
    def __init__(self):
        self.rows = []

    def sample(self, logits, rows):
        self.rows.append([(c.temperature, seed, counter) for c, seed, counter in rows])
        return logits.argmax(dim=-1).tolist()


def make(pool_tokens=64, page=4, batch=4, budget=16, seq=32, policy="on_demand"):
    layout = CacheLayout.from_requirements([PagedKV(1, 16)])
    manager = CacheManager(layout, max_tokens=pool_tokens, page_size=page, max_requests=batch,
                           dtype=torch.float32, device="cpu", max_seq_len=seq)
    model = ScriptedModel()
    runner = StepRunner(model, manager, Runtime(torch.device("cpu"), torch.float32), vocab_size=VOCAB, max_positions=seq)
    sampler = ArgmaxSampler()
    scheduler = Scheduler(runner, sampler, max_batch_size=batch, max_seq_len=seq, eos_token_ids=[EOS],
                          vocab_size=VOCAB, max_tokens_per_step=budget, policy=policy, seed_source=lambda: 77)
    return scheduler, model, manager, sampler


def drain(scheduler, limit=500):
    out = {}
    for _ in range(limit):
        if not scheduler.has_unfinished:
            break
        for index, event in scheduler.step():
            out.setdefault(index, []).append(event)
    assert not scheduler.has_unfinished
    return out


def tokens(events):
    return [e.token_id for e in events if e.token_id is not None]


def test_one_request_prefill_then_single_tokens():
    s, model, manager, _ = make()
    s.add_request([3, 4, 5], max_new_tokens=4)
    out = drain(s)
    assert tokens(out[0]) == [6, 7, 8, 9]
    assert [e.finish_reason for e in out[0]] == [None, None, None, "max_new_tokens"]
    assert out[0][0].prompt_token_count == 3 and out[0][1].prompt_token_count is None
    assert [e.token_index for e in out[0]] == [0, 1, 2, 3]
    assert [b[0] for b in model.batches] == [[3], [1], [1], [1]]   # the last token never pays a decode
    assert manager.active_sequences == 0 and manager.free_pages == manager.num_pages
    manager.check()


def test_prompt_is_cut_under_the_token_budget():
    s, model, _, _ = make(budget=5)
    s.add_request(list(range(10, 23)), max_new_tokens=2)          # 13 tokens -> 5 + 5 + 3
    out = drain(s)
    assert [b[0] for b in model.batches] == [[5], [5], [3], [1]]
    assert model.batches[1][1] == [5, 6, 7, 8, 9]                  # positions continue
    assert tokens(out[0]) == [23, 24]


def test_portions_ride_beside_decoded_tokens():
    s, model, _, _ = make(budget=6)
    s.add_request([1, 2], max_new_tokens=6)
    s.step()                                                      # request 0 is now decoding
    s.add_request(list(range(20, 31)), max_new_tokens=2)          # 11 tokens under what is left of 6
    out = drain(s)
    shapes = [b[0] for b in model.batches]
    assert shapes[1] == [1, 5] and shapes[2] == [1, 5] and shapes[3] == [1, 1]
    assert tokens(out[1]) == [31, 32]


def test_eos_is_emitted_and_stops():
    s, _, manager, _ = make()
    s.add_request([46], max_new_tokens=10)
    out = drain(s)
    assert tokens(out[0]) == [47, 48, 49] and out[0][-1].finish_reason == "eos"
    assert manager.free_pages == manager.num_pages


def test_context_limit_reasons():
    s, model, _, _ = make(seq=8, pool_tokens=64)
    s.add_request([1, 2, 3, 4, 5, 6], max_new_tokens=5)           # room for 2
    s.add_request(list(range(8)), max_new_tokens=3)               # no room at all
    out = drain(s)
    assert tokens(out[0]) == [7, 8] and out[0][-1].finish_reason == "context_length"
    assert out[1][0].token_id is None and out[1][0].finish_reason == "context_length"
    assert out[1][0].prompt_token_count == 8
    assert all(8 not in b[0] for b in model.batches)              # no forward pass for it


def test_add_request_checks():
    s, *_ = make(seq=16, pool_tokens=16)
    with pytest.raises(GenerationError, match="max_new_tokens"):
        s.add_request([1], max_new_tokens=0)
    with pytest.raises(GenerationError, match="context limit"):
        s.add_request([1] * 17, max_new_tokens=1)
    with pytest.raises(GenerationError, match="outside the vocabulary"):
        s.add_request([VOCAB], max_new_tokens=1)
    with pytest.raises(GenerationError, match="at least one token"):
        s.add_request([], max_new_tokens=1)
    with pytest.raises(SamplingError, match="top_k"):
        s.add_request([1], max_new_tokens=1, sampling=SamplingConfig(temperature=1.0, top_k=VOCAB + 1))
    small, *_ = make(seq=32, pool_tokens=16)
    with pytest.raises(GenerationError, match="cache tokens"):
        small.add_request([1] * 10, max_new_tokens=10)


def test_waits_for_a_slot_first_come_first_served():
    s, model, _, _ = make(batch=2)
    for start in (1, 11, 21):
        s.add_request([start], max_new_tokens=3)
    s.step()
    assert s.num_running == 2 and s.num_waiting == 1
    out = drain(s)
    assert tokens(out[2]) == [22, 23, 24]
    joined = [i for i, b in enumerate(model.batches) if b[0] == [1, 1] or b[0] == [1]]
    assert joined                                                 # the third joined once a slot was free


def test_reserve_policy_waits_for_the_whole_lifetime():
    s, model, manager, _ = make(pool_tokens=16, page=4, policy="reserve")
    s.add_request([1, 2, 3], max_new_tokens=9)                    # 12 tokens = 3 pages
    s.add_request([5, 6], max_new_tokens=6)                       # 8 tokens = 2 pages: must wait
    s.step()
    assert s.num_running == 1 and s.num_waiting == 1 and manager.free_pages == 1
    out = drain(s)
    assert tokens(out[1]) == [7, 8, 9, 10, 11, 12]
    assert s.stats["preemptions"] == 0
    manager.check()


def test_pages_run_out_the_last_admitted_is_preempted_and_recomputed():
    s, model, manager, _ = make(pool_tokens=16, page=4, batch=2)
    s.add_request([1, 2, 3, 4, 5, 6], max_new_tokens=9)           # grows to 15 tokens = 4 pages = the pool
    s.add_request([20, 21, 22], max_new_tokens=5)
    out = drain(s)
    assert s.stats["preemptions"] >= 1
    assert tokens(out[0]) == list(range(7, 16))                   # the older request was never disturbed
    assert tokens(out[1]) == [23, 24, 25, 26, 27]                 # recomputed, nothing repeated or lost
    assert [e.token_index for e in out[1]] == [0, 1, 2, 3, 4]
    recomputed = [b for b in model.batches if any(n > 3 for n in b[0][1:])]
    assert recomputed                                             # prompt + generated fed again as one portion
    manager.check()
    assert manager.free_pages == manager.num_pages


def test_failure_releases_everything():
    s, model, manager, _ = make()
    s.add_request([1, 2], max_new_tokens=5)
    s.add_request([3, 4], max_new_tokens=5)
    s.step()
    model.fail_at = len(model.batches)
    with pytest.raises(RuntimeError, match="injected"):
        s.step()
    assert not s.has_unfinished and manager.active_sequences == 0
    assert manager.free_pages == manager.num_pages
    manager.check()


def test_lengths_are_not_committed_by_a_failed_step():
    _, model, manager, _ = make()
    runner = StepRunner(model, manager, Runtime(torch.device("cpu"), torch.float32), vocab_size=VOCAB, max_positions=32)
    from llm_runtime_study_b200.engine.step import StepEntry

    r = manager.admit()
    runner.step([StepEntry(r, [1, 2, 3], [2])])
    assert r.length == 3
    model.fail_at = len(model.batches)
    with pytest.raises(RuntimeError):
        runner.step([StepEntry(r, [4], [0])])
    assert r.length == 3
    with pytest.raises(GenerationError, match="once in a step"):
        runner.step([StepEntry(r, [4], [0]), StepEntry(r, [5], [0])])
    with pytest.raises(GenerationError, match="wanted place"):
        runner.step([StepEntry(r, [4], [1])])
    with pytest.raises(GenerationError, match="exceeds the model limit"):
        runner.step([StepEntry(r, [1] * 30, [])])
    manager.release(r)
    with pytest.raises(KVCacheError, match="released"):
        runner.step([StepEntry(r, [4], [0])])


def test_seeds_and_counters_reach_the_sampler():
    s, _, _, sampler = make()
    s.add_request([1], max_new_tokens=3, sampling=SamplingConfig(temperature=0.7, seed=1234))
    s.add_request([2], max_new_tokens=2)
    drain(s)
    first = [row for rows in sampler.rows for row in rows if row[1] == 1234]
    assert [c for _, _, c in first] == [0, 1, 2] and all(t == 0.7 for t, _, _ in first)
    assert {row[1] for rows in sampler.rows for row in rows} == {1234, 77}


# ------------------------------------------------------------------------------------------------
# Tokens drawn "on the device": the scheduler launches a step and reads its tokens one call later.
# The device side is emulated on the CPU (slot records in a dict, the draw is an argmax), so that
# the scheduler's decisions on this path can be checked without a GPU against the host path above.

class _Handle:
    def __init__(self, ids):
        self._ids = ids

    def tokens(self):
        return list(self._ids)


class EmulatedDeviceRunner(StepRunner):
    """``step_sampled`` / ``decode_sampled`` with the records kept in a dict: token and counter per slot."""

    def __init__(self, *args, **kw):
        super().__init__(*args, **kw)
        self.records = {}
        self.calls = []

    def _draw(self, ctx, entries, drawn):
        logits = self.model.forward(ctx)
        for entry, length in zip(entries, ctx.kv_lens):
            self.manager.commit(entry.request, length)
        ids = logits.argmax(dim=-1).tolist() if logits is not None else []
        for (entry, counter), token in zip(drawn, ids):
            self.records[entry.request.slot] = {"token": token, "counter": counter + 1}
        return _Handle(ids) if drawn else None

    def step_sampled(self, entries, sampler):
        self.calls.append("step")
        ctx = self.build_context(entries)
        return self._draw(ctx, entries, [(e, e.sample.counter) for e in entries if e.sample is not None])

    def decode_sampled(self, requests, sampler):
        from llm_runtime_study_b200.engine.step import StepEntry

        self.calls.append("decode")
        entries = [StepEntry(r, [self.records[r.slot]["token"]], [0]) for r in requests]
        ctx = self.build_context(entries)
        return self._draw(ctx, entries, [(e, self.records[e.request.slot]["counter"]) for e in entries])


class SlotSampler(ArgmaxSampler):
    def sample_slots(self, *args, **kw):        # its presence is what the scheduler looks for
        raise AssertionError("the emulated runner draws by itself")


def make_device(pool_tokens=64, page=4, batch=4, budget=16, seq=32, policy="on_demand", check=None):
    layout = CacheLayout.from_requirements([PagedKV(1, 16)])
    manager = CacheManager(layout, max_tokens=pool_tokens, page_size=page, max_requests=batch,
                           dtype=torch.float32, device="cpu", max_seq_len=seq)
    model = ScriptedModel()
    runner = EmulatedDeviceRunner(model, manager, Runtime(torch.device("cpu"), torch.float32), vocab_size=VOCAB, max_positions=seq)
    scheduler = Scheduler(runner, SlotSampler(), max_batch_size=batch, max_seq_len=seq, eos_token_ids=[EOS],
                          vocab_size=VOCAB, max_tokens_per_step=budget, policy=policy, seed_source=lambda: 77,
                          check_kernels=check)
    assert scheduler.device_sampling
    return scheduler, model, manager, runner


WORKLOAD = [([3, 4, 5], 6), ([46], 10), (list(range(10, 23)), 5), ([7], 1), ([20, 21], 9), ([44, 45, 46], 8)]


@pytest.mark.parametrize("pool,budget,batch", [(64, 16, 4), (24, 5, 3), (40, 7, 2)])
def test_device_path_emits_what_the_host_path_emits(pool, budget, batch):
    outs = []
    for factory in (make, make_device):
        s, model, manager, _ = factory(pool_tokens=pool, budget=budget, batch=batch)
        for prompt, n in WORKLOAD:
            s.add_request(prompt, max_new_tokens=n)
        out = drain(s)
        manager.check()
        assert manager.active_sequences == 0 and manager.free_pages == manager.num_pages
        outs.append({i: [(e.token_id, e.token_index, e.finish_reason, e.prompt_token_count) for e in ev] for i, ev in out.items()})
    assert outs[0] == outs[1]


def test_decode_steps_are_launched_before_the_tokens_of_the_step_before_are_read():
    s, model, manager, runner = make_device()
    s.add_request([3, 4, 5], max_new_tokens=5)
    assert s.step() == []                          # the prompt is launched; its token is not read yet
    first = s.step()                               # nothing but decoding: step 2 is launched, then step 1 read
    assert [e.token_id for _, e in first] == [6] and runner.calls == ["step", "decode"]
    out = drain(s)
    assert tokens(out[0]) == [7, 8, 9, 10] and out[0][-1].finish_reason == "max_new_tokens"
    # five tokens cost one prompt step and four decode steps: the last token never pays a decode, chained or not
    assert runner.calls == ["step"] + ["decode"] * 4 and s.stats["chained_steps"] >= 3


def test_an_eos_found_out_a_step_late_costs_one_dropped_token():
    s, model, manager, runner = make_device()
    s.add_request([46], max_new_tokens=10)         # 47, 48, 49 = EOS
    out = drain(s)
    assert tokens(out[0]) == [47, 48, 49] and out[0][-1].finish_reason == "eos"
    assert runner.calls == ["step", "decode", "decode", "decode"]     # the third decode fed the EOS token: dropped
    assert manager.active_sequences == 0 and manager.free_pages == manager.num_pages
    manager.check()


def test_an_arrival_breaks_the_chain_and_joins():
    s, model, manager, runner = make_device(budget=8)
    s.add_request([1, 2], max_new_tokens=8)
    early = [e.token_id for _ in range(3) for _, e in s.step()]
    s.add_request([30, 31, 32], max_new_tokens=3)
    out = drain(s)
    assert early + tokens(out[0]) == list(range(3, 11)) and tokens(out[1]) == [33, 34, 35]
    assert [1, 3] in [b[0] for b in model.batches]      # the new prompt rode beside a decoded token


def test_a_kernel_that_gave_up_aborts_everything():
    from llm_runtime_study_b200.errors import KernelError

    def check():
        raise KernelError("a bounded wait ran out")

    s, model, manager, _ = make_device(check=check)
    s.add_request([3, 4], max_new_tokens=2)
    s.add_request([9], max_new_tokens=6)
    with pytest.raises(KernelError):
        drain(s)
    assert not s.has_unfinished and manager.active_sequences == 0 and manager.free_pages == manager.num_pages


@pytest.mark.parametrize("factory", [make, make_device])
def test_pages_held_outside_the_scheduler_do_not_make_it_spin(factory):
    s, model, manager, _ = factory(pool_tokens=16, page=4)
    outside = manager.admit()
    manager.grow(outside, 16)                      # the whole pool
    s.add_request([1, 2, 3], max_new_tokens=2)
    with pytest.raises(GenerationError, match="no progress is possible"):
        s.step()
    assert not s.has_unfinished
