"""The cache's bookkeeping (no slot or page lost, held twice or freed twice) and the
generation loop's decisions: the host library's own classes, through its C interface, on the CPU."""
import random

import pytest

from libllm_b200.cache import CacheBook, pool_script
from libllm_b200.engine import SamplingParams, plan_batches, should_stop
from libllm_b200.errors import CacheError, InvalidArgError
from libllm_b200.sampling import uniform


def test_page_pool_never_loses_or_doubles_a_page():
    r = pool_script("pages", 10, [
        dict(op="take", n=4), dict(op="take", n=6), dict(op="take", n=1),           # 0-2
        dict(op="give_back", pages=[0, 1, 2, 3]), dict(op="give_back", pages=[0]),  # 3-4
        dict(op="give_back", pages=[4, 4]), dict(op="give_back", pages=[99]),       # 5-6
        dict(op="check"), dict(op="give_back", pages=[4, 5, 6, 7, 8, 9]), dict(op="check"), dict(op="take", n=10)])
    a, b = r[0]["result"], r[1]["result"]
    assert sorted(a + b) == list(range(10)) and r[1]["available"] == 0
    assert "full" in r[2]["error"]
    assert a == [0, 1, 2, 3] and r[3]["error"] is None
    assert "freed twice" in r[4]["error"] and "twice in one" in r[5]["error"] and "does not exist" in r[6]["error"]
    assert r[6]["available"] == 4 and r[6]["in_use"] == 6       # failed releases changed nothing
    assert r[7]["error"] is None and r[9]["error"] is None
    assert sorted(r[10]["result"]) == list(range(10))


def test_failed_take_takes_nothing():
    r = pool_script("pages", 3, [dict(op="take", n=2), dict(op="take", n=2)])
    assert r[1]["error"] and r[1]["available"] == 1


def test_slots_are_used_again_lowest_first():
    r = pool_script("slots", 3, [dict(op="take"), dict(op="take"), dict(op="take"), dict(op="take"),
                                 dict(op="give_back", slot=1), dict(op="give_back", slot=1), dict(op="take"), dict(op="held")])
    assert [x["result"] for x in r[:3]] == [0, 1, 2]
    assert "no free slot" in r[3]["error"]
    assert r[4]["error"] is None and "freed twice" in r[5]["error"]
    assert r[6]["result"] == 1 and r[7]["result"] == [0, 1, 2]


def full(n_kv=2, d=16):
    return dict(kind="full", n_kv_heads=n_kv, k_dim=d)


def make_cache(capacity=64 * 6, window=None, max_slots=None):
    runs = [full(), dict(kind="window", n_kv_heads=1, k_dim=32, window=window) if window else full(), None]
    return CacheBook(runs, [[], [dict(name="s", shape=[3])], []], capacity, 64, max_slots)


def in_use(cache):
    return [g["pages_in_use"] for g in cache.info()["groups"]]


def test_groups_by_need_and_shared_runs():
    info = make_cache(window=100).info()
    assert len(info["groups"]) == 2 and info["run_group"] == [[0, 0], [1, 0], None]
    same = make_cache().info()
    assert len(same["groups"]) == 1 and same["run_group"] == [[0, 0], [0, 1], None] and same["groups"][0]["runs"] == [0, 1]
    # keys and values of other widths are a need of their own
    wide = CacheBook([full(), dict(kind="full", n_kv_heads=2, k_dim=16, v_dim=40), dict(kind="full", n_kv_heads=2, k_dim=16, v_dim=0)],
                     [], 64).info()
    assert [(g["k_dim"], g["v_dim"]) for g in wide["groups"]] == [(16, 16), (16, 40), (16, 0)]


def test_reserve_is_all_or_nothing_and_close_returns_everything():
    cache = make_cache(capacity=64 * 6)
    a, b = cache.open(), cache.open()
    cache.reserve({a: 100, b: 130})              # 2 + 3 pages
    cache.commit(a, 100)
    cache.commit(b, 130)
    assert in_use(cache) == [5]
    with pytest.raises(CacheError, match="full"):
        cache.reserve({a: 129, b: 200})          # a gets its third page, then b cannot grow
    assert in_use(cache) == [5] and len(cache.info()["sequences"][str(a)]["pages"][0]) == 2
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
    info = cache.info()
    assert in_use(cache) == [0] and info["slots_available"] == info["n_slots"]


def test_window_group_gives_pages_back_as_the_window_moves():
    cache = make_cache(capacity=64 * 8, window=100)
    s = cache.open()
    cache.reserve({s: 300})
    cache.commit(s, 300)                          # later queries see keys >= 300 - 100 + 1 = 201: pages 0..2 go
    pages = cache.info()["sequences"][str(s)]["pages"][1]
    assert pages[:3] == [-1, -1, -1] and pages[3] >= 0
    assert in_use(cache) == [5, 2]
    table = cache.page_table(1, [s], 8)
    assert table.shape == (1, 8) and list(table[0, :3]) == [-1, -1, -1]
    with pytest.raises(CacheError, match="holds 5 pages"):
        cache.page_table(0, [s], 4)
    cache.check()
    cache.close(s)
    cache.check()
    assert in_use(cache) == [0, 0]


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
    assert in_use(cache) == [0, 0]


def test_plan_batches():
    # 64-token pages: requests need 128, 64, 192, 64 tokens of room
    assert plan_batches([100, 10, 150, 5], [20, 20, 20, 20], 256, 8) == [[0, 1], [2, 3]]
    assert plan_batches([100, 10, 150, 5], [20, 20, 20, 20], 1024, 2) == [[0, 1], [2, 3]]
    assert plan_batches([100, 10, 150, 5], [20, 20, 20, 20], 1024, 8) == [[0, 1, 2, 3]]
    assert plan_batches([10], [0], 64, 8) == [[0]]
    assert plan_batches([], [], 64, 8) == []
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
    import numpy as np
    SamplingParams().validate()
    SamplingParams(0.0, 0, 1.0).validate()
    for bad in (SamplingParams(-1.0), SamplingParams(1.0, 5000), SamplingParams(1.0, 50, 0.0), SamplingParams(1.0, 0, 0.5)):
        with pytest.raises(InvalidArgError):
            bad.validate()
    us = [uniform(3, s, t) for s in range(50) for t in range(50)]
    assert all(0.0 <= u < 1.0 for u in us) and abs(sum(us) / len(us) - 0.5) < 0.02
    assert uniform(3, 4, 5) == uniform(3, 4, 5) != uniform(3, 5, 4)
    assert all(float(np.float32(u)) == u for u in us[:100])   # exact in float32
