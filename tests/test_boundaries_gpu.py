"""Places where a size crosses a boundary of the engine: a page, the page table's width (a new
graph), the longest sequence, a launch sequence's token count, and schedules drawn at random on a
small cache.  Every logit is compared with the plain implementation."""
import random

import pytest
import torch

import plain_llama as P
from helpers import check_against_plain, model_folder, plain_weights, tokens_for
from replay import replay_batch

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]
_cache = {}


def setup(name, dtype, **kw):
    from libllm_b200.engine import Engine
    key = (name, dtype, tuple(sorted(kw.items())))
    if key not in _cache:
        folder = model_folder(name)
        kw.setdefault("max_tokens", 4096)
        _cache[key] = (Engine.from_folder(folder, dtype=dtype, **kw), P.read_config(folder), plain_weights(folder))
    return _cache[key]


@pytest.mark.parametrize("dtype", DTYPES)
def test_decoding_across_the_page_tables_width(dtype):
    """Single-token steps from 500 to 530 cached tokens: the ninth page is taken at 512, the page
    table doubles its width and the steps change to another graph."""
    engine, c, w = setup("B", dtype)
    toks = tokens_for("B", 530, 201)
    got = replay_batch(engine, [("r", toks, 500)])["r"]
    check_against_plain(got, c, w, toks, dtype, "across 512 tokens")
    before = engine.info()["graphs_captured"]
    got = replay_batch(engine, [("r", toks, 500)])["r"]          # the same again: every shape is known now
    check_against_plain(got, c, w, toks, dtype, "across 512 tokens, graphs replayed")
    assert engine.info()["graphs_captured"] == before


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n_prompt", [63, 64, 65, 128, 192])
def test_prompts_that_end_at_a_page(n_prompt, dtype):
    engine, c, w = setup("C", dtype)
    toks = tokens_for("C", n_prompt + 3, 210 + n_prompt)
    got = replay_batch(engine, [("r", toks, n_prompt)])["r"]
    check_against_plain(got, c, w, toks, dtype, f"prompt of {n_prompt}")


def test_the_longest_sequence_and_one_token_more():
    """A sequence may grow to max_seq_len and not beyond; the refusal changes nothing."""
    from libllm_b200.engine import StepItem
    from libllm_b200.errors import InvalidArgError
    engine, c, w = setup("A", "float32", max_seq_len=130, max_tokens=512)
    toks = tokens_for("A", 130, 220)
    s = engine.open_sequence()
    rows = [torch.from_numpy(engine.step([StepItem(s, toks[:127], list(range(127)))]))]
    for t in toks[127:]:
        rows.append(torch.from_numpy(engine.step([StepItem(s, [t], [0])])))
    check_against_plain(torch.cat(rows), c, w, toks, "float32", "up to the longest sequence")
    pages = engine.pages_in_use()
    with pytest.raises(InvalidArgError):
        engine.step([StepItem(s, [1], [0])])
    assert engine.pages_in_use() == pages and engine.sequence_length(s) == 130
    engine.close_sequence(s)
    assert engine.pages_in_use() == [0]
    engine.cache_check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("seed", [1, 2, 3])
def test_schedules_drawn_at_random_on_a_small_cache(seed, dtype):
    """Batches of one to five requests with prompt lengths from 1 to 150 and 1 to 20 further tokens,
    one batch after another on a cache that holds little more than one of them, launch sequences of
    at most 96 tokens: every request's logits are the plain implementation's."""
    rng = random.Random(seed)
    engine, c, w = setup("B", dtype, max_tokens=1024, max_step_tokens=96)
    for b in range(4):
        reqs = []
        for j in range(rng.randint(1, 5)):
            n_prompt, n_more = rng.randint(1, 150), rng.randint(1, 20)
            reqs.append((f"s{seed}b{b}r{j}", tokens_for("B", n_prompt + n_more, 1000 * seed + 10 * b + j), n_prompt))
        got = replay_batch(engine, reqs)
        for rid, toks, _ in reqs:
            check_against_plain(got[rid], c, w, toks, dtype, rid)
        assert engine.pages_in_use() == [0]
    engine.cache_check()
