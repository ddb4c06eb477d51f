"""The cache's bookkeeping (no slot or page lost, held twice or freed twice) and the
generation loop's decisions, on the host."""
import random

import pytest
import torch

from libllm_b200.cache import KVCache, PagePool, SlotTable
from libllm_b200.engine.generate import plan_batches, should_stop
from libllm_b200.engine.step import SamplingParams
from libllm_b200.errors import CacheError, InvalidArgError
from libllm_b200.parts.base import CacheNeed, StateNeed
from libllm_b200.sampling import uniform


def test_page_pool_never_loses_or_doubles_a_page():
    pool = PagePool(10)
    a = pool.take(4)
    b = pool.take(6)
    assert sorted(a + b) == list(range(10)) and pool.available == 0
    with pytest.raises(CacheError, match="full"):
        pool.take(1)
    pool.give_back(a)
    with pytest.raises(CacheError, match="freed twice"):
        pool.give_back([a[0]])
    with pytest.raises(CacheError, match="twice in one"):
        pool.give_back([b[0], b[0]])
    with pytest.raises(CacheError, match="does not exist"):
        pool.give_back([99])
    assert pool.available == 4 and pool.in_use == 6       # failed releases changed nothing
    pool.check()
    pool.give_back(b)
    pool.check()
    assert sorted(pool.take(10)) == list(range(10))


def test_failed_take_takes_nothing():
    pool = PagePool(3)
    pool.take(2)
    with pytest.raises(CacheError):
        pool.take(2)
    assert pool.available == 1


def test_slots_are_used_again_lowest_first():
    slots = SlotTable(3)
    a, b, c = slots.take(), slots.take(), slots.take()
    assert (a, b, c) == (0, 1, 2)
    with pytest.raises(CacheError, match="no free slot"):
        slots.take()
    slots.give_back(b)
    with pytest.raises(CacheError, match="freed twice"):
        slots.give_back(b)
    assert slots.take() == 1 and slots.held() == [0, 1, 2]


def make_cache(capacity=64 * 6, window=None, max_slots=None):
    needs = [CacheNeed("full", 2, 16), CacheNeed("window", 1, 32, window) if window else CacheNeed("full", 2, 16), None]
    states = [{}, {"s": StateNeed((3,))}, {}]
    return KVCache(needs, states, capacity, torch.float32, "cpu", page_size=64, max_slots=max_slots, allocate=False)


def test_groups_by_need_and_shared_runs():
    cache = make_cache(window=100)
    assert len(cache.groups) == 2 and cache.run_group == [(0, 0), (1, 0), None]
    same = make_cache()
    assert len(same.groups) == 1 and same.run_group == [(0, 0), (0, 1), None] and same.groups[0].runs == [0, 1]


def test_reserve_is_all_or_nothing_and_close_returns_everything():
    cache = make_cache(capacity=64 * 6)
    a, b = cache.open(), cache.open()
    cache.reserve({a: 100, b: 130})              # 2 + 3 pages
    cache.commit(a, 100)
    cache.commit(b, 130)
    assert cache.groups[0].pool.in_use == 5
    with pytest.raises(CacheError, match="full"):
        cache.reserve({a: 129, b: 200})          # a gets its third page, then b cannot grow
    assert cache.groups[0].pool.in_use == 5 and len(cache.sequences[a].pages[0]) == 2
    cache.check()
    with pytest.raises(CacheError, match="shrink"):
        cache.reserve({a: 50})
    cache.close(a)
    with pytest.raises(CacheError, match="not open"):
        cache.close(a)
    with pytest.raises(CacheError, match="not open"):
        cache.reserve({a: 10})
    c = cache.open()
    assert c == a                                 # the slot is used again
    cache.reserve({c: 64 * 3})
    cache.check()
    cache.close(b)
    cache.close(c)
    cache.check()
    assert cache.groups[0].pool.in_use == 0 and cache.slots.available == cache.slots.n_slots


def test_window_group_gives_pages_back_as_the_window_moves():
    cache = make_cache(capacity=64 * 8, window=100)
    s = cache.open()
    cache.reserve({s: 300})
    cache.commit(s, 300)                          # later queries see keys >= 300 - 100 + 1 = 201: pages 0..2 go
    assert cache.sequences[s].pages[1][:4] == [-1, -1, -1, cache.sequences[s].pages[1][3]]
    assert cache.groups[1].pool.in_use == 2 and cache.groups[0].pool.in_use == 5
    table = cache.page_table(1, [s], 8)
    assert table.shape == (1, 8) and list(table[0, :3]) == [-1, -1, -1]
    cache.check()
    cache.close(s)
    cache.check()
    assert cache.groups[1].pool.in_use == 0


def test_random_walk_keeps_the_books_consistent():
    rng = random.Random(0)
    cache = make_cache(capacity=64 * 20, window=70, max_slots=6)
    live = {}
    for _ in range(600):
        r = rng.random()
        try:
            if r < 0.25 and len(live) < 6:
                live[cache.open()] = 0
            elif r < 0.45 and live:
                s = rng.choice(list(live))
                cache.close(s)
                del live[s]
            elif live:
                s = rng.choice(list(live))
                n = live[s] + rng.randint(1, 150)
                cache.reserve({s: n})
                cache.commit(s, n)
                live[s] = n
        except CacheError as e:
            assert "full" in str(e) or "no free slot" in str(e)
        cache.check()
    for s in list(live):
        cache.close(s)
    cache.check()
    assert all(g.pool.in_use == 0 for g in cache.groups)


def test_state_is_zeroed_when_a_slot_is_used_again():
    needs = [CacheNeed("full", 1, 16)]
    cache = KVCache(needs, [{"h": StateNeed((4,))}], 128, torch.float32, "cpu", max_slots=2)
    s = cache.open()
    cache.state[0]["h"][s] += 5
    cache.close(s)
    s2 = cache.open()
    assert s2 == s and float(cache.state[0]["h"][s2].abs().sum()) == 0


def test_plan_batches():
    # 64-token pages: requests need 128, 64, 192, 64 tokens of room
    assert plan_batches([100, 10, 150, 5], [20, 20, 20, 20], 256, 8) == [[0, 1], [2, 3]]
    assert plan_batches([100, 10, 150, 5], [20, 20, 20, 20], 1024, 2) == [[0, 1], [2, 3]]
    assert plan_batches([100, 10, 150, 5], [20, 20, 20, 20], 1024, 8) == [[0, 1, 2, 3]]
    assert plan_batches([10], [0], 64, 8) == [[0]]
    with pytest.raises(CacheError, match="needs room"):
        plan_batches([300], [10], 256, 8)
    with pytest.raises(InvalidArgError, match="at least one token"):
        plan_batches([0], [10], 256, 8)
    with pytest.raises(InvalidArgError, match="longest"):
        plan_batches([100], [100], 1024, 8, max_seq_len=150)


def test_should_stop():
    assert should_stop(7, 0, 10, {7}) == (True, False)           # a stop token ends and is not handed out
    assert should_stop(5, 0, 10, {7}) == (False, True)
    assert should_stop(5, 9, 10, {7}) == (True, True)            # the last allowed token is handed out
    assert should_stop(7, 9, 10, {7}) == (True, False)


def test_sampling_params_and_uniforms():
    SamplingParams().validate()
    SamplingParams(0.0, 0, 1.0).validate()
    for bad in (SamplingParams(-1.0), SamplingParams(1.0, 5000), SamplingParams(1.0, 50, 0.0), SamplingParams(1.0, 0, 0.5)):
        with pytest.raises(InvalidArgError):
            bad.validate()
    us = [uniform(3, s, t) for s in range(50) for t in range(50)]
    assert all(0.0 <= u < 1.0 for u in us) and abs(sum(us) / len(us) - 0.5) < 0.02
    assert uniform(3, 4, 5) == uniform(3, 4, 5) != uniform(3, 5, 4)
    assert all(float(torch.tensor(u, dtype=torch.float32)) == u for u in us[:100])   # exact in float32
