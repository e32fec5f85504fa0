"""Page accounting of the cache manager (no GPU): no page lost, held twice or
freed twice, under random orders of requests; windows; slots."""

import random

import pytest
import torch

from llm_runtime_study_b200.cache import CacheLayout, CacheManager, PageAllocator
from llm_runtime_study_b200.errors import KVCacheError
from llm_runtime_study_b200.parts.base import FixedState, PagedKV


def _manager(max_tokens=64, page=4, requests=4, window=None, extra=()):
    needs = [PagedKV(2, 16), PagedKV(2, 16), *extra]
    if window:
        needs.append(PagedKV(2, 16, window=window))
    layout = CacheLayout.from_requirements(needs)
    return CacheManager(layout, max_tokens=max_tokens, page_size=page, max_requests=requests,
                        dtype=torch.float32, device="cpu")


def test_allocator_lowest_first_and_double_free():
    a = PageAllocator(4)
    assert a.allocate(2) == [0, 1]
    a.free([0])
    assert a.allocate(2) == [0, 2]
    with pytest.raises(KVCacheError, match="exhausted: need 2 pages but only 1"):
        a.allocate(2)
    with pytest.raises(KVCacheError, match="not held"):
        a.free([3])
    a.free([1])
    with pytest.raises(KVCacheError, match="not held"):
        a.free([1])
    with pytest.raises(KVCacheError, match="twice"):
        a.free([0, 0])
    a.check()


def test_layers_with_equal_needs_share_a_group():
    layout = CacheLayout.from_requirements(
        [PagedKV(2, 16), PagedKV(2, 16, window=8), None, PagedKV(2, 16), FixedState((5,))])
    assert [g.layers for g in layout.groups] == [(0, 3), (1,)]
    assert [s.layer for s in layout.states] == [4]


def test_grow_commit_release_and_reuse():
    m = _manager(max_tokens=32, page=4)
    r = m.admit()
    m.grow(r, 7)
    assert r.tables[0] == [0, 1] and r.length == 0
    m.commit(r, 7)
    m.grow(r, 8)
    assert r.tables[0] == [0, 1]            # still fits
    m.grow(r, 9)
    assert r.tables[0] == [0, 1, 2]
    with pytest.raises(KVCacheError, match="exceeds"):
        m.commit(r, 13)
    r2 = m.admit()
    m.grow(r2, 4)
    assert r2.tables[0] == [3]
    m.release(r)
    m.release(r)                             # idempotent
    with pytest.raises(KVCacheError, match="released"):
        m.grow(r, 1)
    r3 = m.admit()
    m.grow(r3, 12)
    assert r3.tables[0] == [0, 1, 2]        # lowest ids come back first
    m.check()
    assert m.used_tokens == 0 and m.active_sequences == 2


def test_exhaustion_takes_nothing():
    m = _manager(max_tokens=16, page=4)
    a, b = m.admit(), m.admit()
    m.grow(a, 12)
    with pytest.raises(KVCacheError, match="need 2 pages but only 1"):
        m.grow(b, 8)
    assert b.tables[0] == [] and m.free_pages == 1
    assert not m.can_grow(b, 8) and m.can_grow(b, 4)
    m.check()


def test_slots_run_out_and_state_is_zeroed():
    m = _manager(requests=2, extra=(FixedState((3,)),))
    a, b = m.admit(), m.admit()
    with pytest.raises(KVCacheError, match="slots"):
        m.admit()
    state = m.layer_cache(2).state
    assert state.shape == (2 + 1, 3)          # one row per request slot and the row of the padding slot
    assert m.padding_slot == 2 and m.slots.records.shape == (3, 12)
    state[a.slot] = 7.0
    m.release(a)
    c = m.admit()
    assert c.slot == a.slot and float(state[c.slot].abs().sum()) == 0.0
    m.check()


def test_window_gives_pages_back_early():
    m = _manager(max_tokens=64, page=4, window=6)
    r = m.admit()
    m.grow(r, 20)
    m.commit(r, 20)
    full, windowed = r.tables
    assert full == [0, 1, 2, 3, 4]
    # next query at position 20 reads keys 15..20: pages 0..2 (keys 0..11) are dead
    assert windowed == [-1, -1, -1, 3, 4]
    assert m.allocators[1].num_free == m.num_pages - 2
    m.grow(r, 24)
    assert r.tables[1][-1] == 0              # a returned page is used again
    m.check()
    m.release(r)
    m.check()
    assert m.allocators[1].num_free == m.num_pages


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_keep_the_books(seed):
    rng = random.Random(seed)
    m = _manager(max_tokens=96, page=4, requests=5, window=10)
    live = []
    for _ in range(400):
        action = rng.random()
        if action < 0.25 and m.free_slots:
            live.append(m.admit())
        elif action < 0.8 and live:
            r = rng.choice(live)
            target = r.length + rng.randint(1, 9)
            if m.can_grow(r, target):
                m.grow(r, target)
                if rng.random() < 0.9:      # a failed step commits nothing
                    m.commit(r, target)
            else:
                with pytest.raises(KVCacheError):
                    m.grow(r, target)
        elif live:
            r = live.pop(rng.randrange(len(live)))
            m.release(r)
            if rng.random() < 0.3:
                m.release(r)
        m.check()
    for r in live:
        m.release(r)
    m.check()
    assert all(a.num_free == m.num_pages for a in m.allocators) and m.free_slots == 5


def test_groups_with_their_own_tensors_page_size_and_window_pool():
    """A group states its tensors per token and may bring a page size of its own; a group that reads a window
    only gets a pool for the window (and one step's tokens), not for whole sequences."""

    from llm_runtime_study_b200.cache.manager import pool_shape
    from llm_runtime_study_b200.parts.base import PagedTensors

    latent = PagedTensors(tensors=(("latent", (24,)), ("rope_key", (1, 8))), page_size=8)
    windowed = PagedKV(2, 16, window=12)
    layout = CacheLayout.from_requirements([PagedKV(2, 16), latent, windowed, latent])
    m = CacheManager(layout, max_tokens=256, page_size=4, max_requests=3, dtype=torch.float32, device="cpu",
                     max_seq_len=128, max_step_tokens=16)
    full, lat, win = m.groups
    assert (full.page_size, full.num_pages) == (4, 64) and (lat.page_size, lat.num_pages) == (8, 32)
    assert win.num_pages == 3 * (3 + 3) + 4 < full.num_pages          # window of 12 = 3 pages, +3 per request, +16 tokens
    assert lat.tensors["latent"].shape == (2, 32, 8, 24) and lat.tensors["rope_key"].shape == (2, 32, 1, 8, 8)
    assert pool_shape((2, 16), 5, 4) == (5, 2, 4, 16) and pool_shape((24,), 5, 8) == (5, 8, 24)
    view = m.layer_cache(3)
    assert view.page_size == 8 and set(view.tensors) == {"latent", "rope_key"} and view.keys is None
    assert m.layer_cache(0).keys.shape == (64, 2, 4, 16) and m.max_request_tokens == 256
    # a request grows in every group by that group's own pages
    r = m.admit()
    m.grow(r, 21)
    assert [len(t) for t in r.tables] == [6, 3, 6]
    m.commit(r, 21)
    assert r.tables[2][:2] == [-1, -1] and r.tables[2][2] >= 0         # positions 0..7 lie behind the window of 12
    budget = m.budget()
    assert budget.free == [58, 29, win.num_pages - 4]
    assert budget.room(m.held(r)) == min(64 * 4, 32 * 8, (6 + win.num_pages - 4) * 4)
    assert budget.take(m.held(r), 40) and budget.free == [54, 27, win.num_pages - 8]
    assert not budget.take(m.held(None) or [0, 0, 0], 10_000)
    m.release(r)
    m.check()
    assert m.all_free


def test_a_long_request_lives_in_a_window_pool_that_is_much_smaller_than_it():
    layout = CacheLayout.from_requirements([PagedKV(1, 16, window=8)])
    m = CacheManager(layout, max_tokens=4096, page_size=4, max_requests=2, dtype=torch.float32, device="cpu",
                     max_seq_len=4096, max_step_tokens=8)
    assert m.groups[0].num_pages == 2 * (2 + 3) + 2 and m.max_request_tokens == 4096
    r = m.admit()
    length = 0
    while length < 4000:
        step = min(8, 4000 - length)
        m.grow(r, length + step)
        length += step
        m.commit(r, length)
        m.check()
    assert m.groups[0].allocator.num_held <= 4
    m.release(r)
    assert m.all_free
