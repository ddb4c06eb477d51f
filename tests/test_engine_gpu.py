"""The engine against the plain implementation, in float32 and bfloat16, for every way of
cutting the work: whole requests, the last 32 tokens one by one, batches of unequal
lengths whose shorter requests end earlier with slots used again, long decoding, and the
first tokens of a sequence."""
import pytest
import torch

import plain_llama as P
from helpers import check_against_plain, check_logits, model_folder, plain_weights, tokens_for
from replay import replay_batch

pytestmark = pytest.mark.gpu

DTYPES = ["float32", "bfloat16"]
_cache = {}


def setup(name, dtype, max_tokens=4096, **kw):
    from libllm_b200.engine import Engine
    key = (name, dtype, max_tokens, tuple(sorted(kw.items())))
    if key not in _cache:
        folder = model_folder(name)
        _cache[key] = (Engine.from_folder(folder, dtype=dtype, max_tokens=max_tokens, **kw), P.read_config(folder),
                       plain_weights(folder))
    return _cache[key]


def plain(c, w, toks):
    return P.forward_logits(c, w, toks)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_each_request_alone_and_whole(name, dtype):
    engine, c, w = setup(name, dtype)
    for i, n in enumerate([1, 2, 5, 33, 64, 65, 131]):
        toks = tokens_for(name, n, i)
        got = replay_batch(engine, [("r", toks, n)])["r"]
        check_against_plain(got, c, w, toks, dtype, f"{name} whole len {n}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_prompts_of_hundreds_of_tokens(name, dtype):
    """Prompt steps above the token count where the products change hands (the library's product,
    which adds its result to the residual stream as it stores): one prompt alone, then two of unequal
    lengths in one step, each followed by a few single tokens."""
    engine, c, w = setup(name, dtype)
    toks = tokens_for(name, 420, 61)
    got = replay_batch(engine, [("r", toks, 417)])["r"]
    check_against_plain(got, c, w, toks, dtype, f"{name} prompt of 417")
    reqs = [("long", tokens_for(name, 303, 62), 300), ("short", tokens_for(name, 95, 63), 90)]
    got = replay_batch(engine, reqs)
    for rid, toks, _ in reqs:
        check_against_plain(got[rid], c, w, toks, dtype, f"{name} {rid} beside the other")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_last_32_tokens_one_by_one(name, dtype):
    engine, c, w = setup(name, dtype)
    for i, n in enumerate([33, 100, 160]):
        toks = tokens_for(name, n, 10 + i)
        got = replay_batch(engine, [("r", toks, n - 32)])["r"]
        check_against_plain(got, c, w, toks, dtype, f"{name} last-32 len {n}")


WORKLOADS = {
    # (prompt lengths, decoded tokens): the two tiny workloads of the benchmark description
    "A": ([5, 9, 12], 8),
    "B": ([1, 7, 33, 70], 16),
    "C": ([3, 64, 17], 5),
}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_unequal_batches_one_after_another(name, dtype):
    """Three batches on a cache that holds only one of them at a time: slots and pages
    are used again.  Requests decode different numbers of tokens, so some end earlier."""
    prompts, n_dec = WORKLOADS[name]
    cap = sum((p + n_dec + len(prompts) + 63) // 64 * 64 for p in prompts)
    engine, c, w = setup(name, dtype, max_tokens=cap)
    for b in range(3):
        reqs = []
        for j, p in enumerate(prompts):
            total = p + n_dec - (j if b % 2 == 0 else len(prompts) - 1 - j)   # unequal ends
            reqs.append((f"b{b}r{j}", tokens_for(name, total, 100 * b + j), p))
        got = replay_batch(engine, reqs)
        for rid, toks, _ in reqs:
            check_against_plain(got[rid], c, w, toks, dtype, f"{name} batch {b} {rid}")
    assert engine.pages_in_use() == [0]


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding(dtype):
    """One token a step for 300 steps after a one-token prompt: crosses several pages."""
    engine, c, w = setup("B", dtype)
    toks = tokens_for("B", 300, 77)
    got = replay_batch(engine, [("r", toks, 1)])["r"]
    check_against_plain(got, c, w, toks, dtype, "long decoding")


@pytest.mark.parametrize("dtype", DTYPES)
def test_first_tokens_of_a_sequence(dtype):
    """Positions 0, 1, 2 of short sequences, alone and beside a long neighbour."""
    engine, c, w = setup("A", dtype)
    short = tokens_for("A", 3, 5)
    long_ = tokens_for("A", 90, 6)
    alone = replay_batch(engine, [("s", short, 1)])["s"]
    both = replay_batch(engine, [("l", long_, 60), ("s", short, 1)])
    check_against_plain(alone, c, w, short, dtype, "first tokens alone")
    check_against_plain(both["s"], c, w, short, dtype, "first tokens beside a long request")
    check_against_plain(both["l"], c, w, long_, dtype, "long neighbour")


@pytest.mark.parametrize("dtype", DTYPES)
def test_prompt_cut_into_chunks(dtype):
    """A step with more tokens than one launch sequence takes is cut inside a prompt."""
    engine, c, w = setup("C", dtype, max_step_tokens=48)
    reqs = [("a", tokens_for("C", 100, 1), 100), ("b", tokens_for("C", 30, 2), 30)]
    got = replay_batch(engine, reqs)
    for rid, toks, _ in reqs:
        check_against_plain(got[rid], c, w, toks, dtype, f"chunked {rid}")
    # a prompt whose pages outnumber the page table of its first launch sequences (the step takes all
    # its pages before the first of them runs)
    toks = tokens_for("C", 702, 3)
    got = replay_batch(engine, [("long", toks, 700)])["long"]
    check_against_plain(got, c, w, toks, dtype, "chunked prompt of 700")


def test_batch_composition_does_not_change_float32_results():
    """The same request alone and in a batch: float32 logits agree to rounding."""
    engine, c, w = setup("B", "float32")
    t0, t1, t2 = (tokens_for("B", n, 40 + n) for n in (50, 7, 90))
    alone = replay_batch(engine, [("x", t0, 40)])["x"]
    batch = replay_batch(engine, [("y", t1, 3), ("x", t0, 40), ("z", t2, 80)])["x"]
    assert float((alone - batch).abs().max()) <= 1e-6 * float(alone.abs().mean()) + 1e-7


def test_errors_leave_the_cache_unchanged():
    from libllm_b200.engine import StepItem
    from libllm_b200.errors import CacheError, InvalidArgError
    engine, c, w = setup("A", "float32", max_tokens=128)
    s = engine.open_sequence()
    with pytest.raises(InvalidArgError):
        engine.step([StepItem(s, [1, 2, 999], [0])])           # token outside the vocabulary
    with pytest.raises(InvalidArgError):
        engine.step([StepItem(s, [1, 2], [5])])                # wanted place outside the tokens
    s2 = engine.open_sequence()
    with pytest.raises(CacheError):
        engine.step([StepItem(s, [1] * 100, []), StepItem(s2, [1] * 100, [])])   # 4 pages wanted, 2 exist
    assert engine.pages_in_use() == [0]
    engine.cache_check()
    engine.close_sequence(s)
    engine.close_sequence(s2)
    with pytest.raises(CacheError):
        engine.close_sequence(s2)


@pytest.mark.parametrize("dtype", DTYPES)
def test_prompt_steps_of_a_repeating_shape_stay_right(dtype):
    """Batches of the same shape (tokens, sequences, wanted places) but with the tokens spread
    differently over the sequences, standing behind different numbers of cached tokens: the step's
    buffers are used again from batch to batch, what each sequence has is in the descriptor."""
    from libllm_b200.engine import StepItem
    engine, c, w = setup("B", dtype, max_tokens=8192)
    rounds = [[20, 50, 7], [7, 20, 50], [30, 30, 17], [50, 7, 20], [25, 26, 26]]
    for r, lens in enumerate(rounds):
        seqs = [tokens_for("B", n, 100 + 10 * r + i) for i, n in enumerate(lens)]
        slots = [engine.open_sequence() for _ in seqs]
        logits = torch.from_numpy(engine.step([StepItem(s, t, [0, len(t) - 1]) for s, t in zip(slots, seqs)]))
        # a second step of the same sequences, eight tokens each behind what is cached now
        more = [tokens_for("B", 8, 500 + 10 * r + i) for i in range(len(seqs))]
        logits2 = torch.from_numpy(engine.step([StepItem(s, t, [7]) for s, t in zip(slots, more)]))
        for s in slots:
            engine.close_sequence(s)
        for i, t in enumerate(seqs):
            ref = plain(c, w, t + more[i])
            check_logits(logits[2 * i:2 * i + 2], ref[[0, len(t) - 1]], dtype, f"round {r} sequence {i}")
            check_logits(logits2[i:i + 1], ref[[len(t) + 7]], dtype, f"round {r} sequence {i}, second step")


def test_wanted_places_in_any_order_across_pieces():
    """``want`` need not ascend, and a prompt cut into pieces still hands its rows back in the
    order asked for."""
    from libllm_b200.engine import StepItem
    engine, c, w = setup("C", "float32", max_step_tokens=48)
    a, b = tokens_for("C", 100, 21), tokens_for("C", 30, 22)
    sa, sb = engine.open_sequence(), engine.open_sequence()
    got = torch.from_numpy(engine.step([StepItem(sa, a, [99, 3, 50]), StepItem(sb, b, [29, 0])]))
    engine.close_sequence(sa)
    engine.close_sequence(sb)
    check_logits(got[:3], plain(c, w, a)[[99, 3, 50]], "float32", "rows of a")
    check_logits(got[3:], plain(c, w, b)[[29, 0]], "float32", "rows of b")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B"])
def test_a_prompt_whose_last_row_alone_is_wanted(name, dtype):
    """The step a generation starts with: the last layer then runs its feed-forward for the wanted
    rows alone.  One row, a row wanted twice beside others, and two prompts of unequal lengths; then a
    token more for each, which reads the keys and values the prompt step left in every layer."""
    from libllm_b200.engine import StepItem
    engine, c, w = setup(name, dtype)
    a, b = tokens_for(name, 301, 71), tokens_for(name, 41, 72)
    ref_a, ref_b = plain(c, w, a), plain(c, w, b)
    sa, sb = engine.open_sequence(), engine.open_sequence()
    got = torch.from_numpy(engine.step([StepItem(sa, a[:300], [299]), StepItem(sb, b[:40], [39, 7, 39])]))
    check_logits(got[:1], ref_a[[299]], dtype, "last row of a")
    check_logits(got[1:], ref_b[[39, 7, 39]], dtype, "rows of b")
    got = torch.from_numpy(engine.step([StepItem(sa, a[300:], [0]), StepItem(sb, b[40:], [0])]))
    check_logits(got[:1], ref_a[[300]], dtype, "a's next token")
    check_logits(got[1:], ref_b[[40]], dtype, "b's next token")
    engine.close_sequence(sa)
    engine.close_sequence(sb)
    # the same prompt cut into launch sequences of 48 tokens: the first six want nothing at all
    engine, c, w = setup(name, dtype, max_step_tokens=48)
    sa = engine.open_sequence()
    got = torch.from_numpy(engine.step([StepItem(sa, a[:300], [299])]))
    check_logits(got, ref_a[[299]], dtype, "last row of a, cut")
    got = torch.from_numpy(engine.step([StepItem(sa, a[300:], [0])]))
    check_logits(got, ref_a[[300]], dtype, "a's next token, cut")
    engine.close_sequence(sa)


@pytest.mark.parametrize("dtype", DTYPES)
def test_tensors_stored_in_other_types_load_to_the_same_model(dtype):
    """Weights handed over in host memory as bfloat16, float32 or float64 (the same values) are
    converted by role: operands of products to the engine's type, norm weights to 32-bit."""
    from libllm_b200.engine import Engine, StepItem
    folder = model_folder("A")
    w = plain_weights(folder)                                  # float64, the stored bfloat16 values
    toks = tokens_for("A", 40, 31)
    outs = []
    for conv in (lambda t: t.to(torch.bfloat16), lambda t: t.float(), lambda t: t.double().numpy(), lambda t: t.float().numpy()):
        engine = Engine.from_tensors(P.read_config(folder) | {"model_type": "llama"}, {k: conv(v) for k, v in w.items()},
                                     dtype=dtype, max_tokens=128)
        s = engine.open_sequence()
        outs.append(torch.from_numpy(engine.step([StepItem(s, toks, [0, 20, 39])])))
        engine.close()
    for o in outs[1:]:
        assert torch.equal(o, outs[0])
    check_logits(outs[0], plain(P.read_config(folder), w, toks)[[0, 20, 39]], dtype, "from tensors in host memory")
    # the folder's own loader gives the same
    engine, _, _ = setup("A", dtype)
    s = engine.open_sequence()
    assert torch.equal(torch.from_numpy(engine.step([StepItem(s, toks, [0, 20, 39])])), outs[0])
    engine.close_sequence(s)
