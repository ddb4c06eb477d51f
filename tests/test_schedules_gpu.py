"""The schedules the benchmark times, and the same batches over and over.

* The benchmark's own shapes through the engine against the plain implementation: the real
  vocabulary (128,256: a thousand tiles of the output matrix's product, 32-bit logit rows), prompts
  of 2,048 tokens (sixteen query tiles by thirty-two key tiles per head inside a step, a step of
  16,384 tokens cut into two pieces), single-token steps through captured graphs at page tables 64
  wide with 8 and 64 sequences (key splits joined, products cut along K).  Two layers keep the plain
  implementation affordable; every kernel shape of a layer is the full-size one.
* Two unequal batches back to back a hundred times on one engine, with captured graphs taking
  turns and slots used again, against the same trace on an engine that captures nothing: in
  float32 bit for bit, in bfloat16 within the usual bounds."""
import pytest
import torch

import plain_llama as P
from helpers import check_logits, model_folder, plain_weights, rel_err, rms_err, tokens_for
from replay import replay_batch

pytestmark = pytest.mark.gpu

BENCH_SIZES = dict(model_type="llama", num_hidden_layers=2, hidden_size=2048, num_attention_heads=32,
                   num_key_value_heads=8, head_dim=64, intermediate_size=8192, vocab_size=128256,
                   rope_theta=500000.0,
                   rope_scaling=dict(rope_type="llama3", factor=32.0, low_freq_factor=1.0, high_freq_factor=4.0,
                                     original_max_position_embeddings=8192),
                   rms_norm_eps=1e-5, tie_word_embeddings=True, max_position_embeddings=131072, hidden_act="silu")
_state = {}


def bench_model():
    if not _state:
        folder = model_folder("bench_sizes", seed=21, config=BENCH_SIZES)
        _state.update(folder=folder, c=P.read_config(folder), w=plain_weights(folder))
    return _state["folder"], _state["c"], _state["w"]


def check_rows_against_the_floor(got, c, w, toks, rows, what):
    """bfloat16 at these sizes: within twice the distance between the plain implementation with
    activations rounded to bfloat16 where an engine must round them and its exact form."""
    exact = P.forward_logits(c, w, toks, rows=rows)
    rounded = P.forward_logits(c, w, toks, act_dtype=torch.bfloat16, rows=rows)
    floor_max, floor_rms = rel_err(rounded, exact), rms_err(rounded, exact)
    e, r = rel_err(got, exact), rms_err(got, exact)
    assert torch.isfinite(got).all(), what
    assert e < 2 * floor_max, f"{what}: rel err {e:.3e}, the rounding floor is {floor_max:.3e}"
    assert r < 2 * floor_rms, f"{what}: rms err {r:.3e}, the rounding floor is {floor_rms:.3e}"
    top2 = exact.topk(2, dim=-1).values
    clear = (top2[..., 0] - top2[..., 1]) > 4 * floor_max * float(exact.abs().mean())
    assert bool(((got.argmax(-1) == exact.argmax(-1)) | ~clear).all()), f"{what}: argmax differs where the margin is clear"


def run_prompts_then_single_tokens(engine, seqs, n_prompt, n_single):
    """Every sequence's first ``n_prompt[i]`` tokens in ONE step (the last row wanted), then
    ``n_single`` steps of one token each; returns per sequence the 1 + n_single wanted rows."""
    from libllm_b200.engine import StepItem
    slots = [engine.open_sequence() for _ in seqs]
    rows = [[] for _ in seqs]
    first = torch.from_numpy(engine.step([StepItem(s, t[:n], [n - 1]) for s, t, n in zip(slots, seqs, n_prompt)]))
    for i in range(len(seqs)):
        rows[i].append(first[i:i + 1])
    for k in range(n_single):
        out = torch.from_numpy(engine.step([StepItem(s, [t[n + k]], [0]) for s, t, n in zip(slots, seqs, n_prompt)]))
        for i in range(len(seqs)):
            rows[i].append(out[i:i + 1])
    for s in slots:
        engine.close_sequence(s)
    engine.cache_check()
    return [torch.cat(r) for r in rows]


def test_the_benchmarks_decode_schedule_eight_prompts_of_2048():
    from libllm_b200.engine import Engine
    folder, c, w = bench_model()
    engine = Engine.from_folder(folder, dtype="bfloat16", max_tokens=8 * 2112, max_seq_len=4096)
    g = torch.Generator().manual_seed(5)
    seqs = [torch.randint(0, 128256, (2052,), generator=g).tolist() for _ in range(8)]
    got = run_prompts_then_single_tokens(engine, seqs, [2048] * 8, 4)
    info = engine.info()
    assert info["graphs_captured"] == 2 and info["graph_replays"] == 2          # two graphs of the shape take turns
    for i in (0, 5, 7):
        check_rows_against_the_floor(got[i], c, w, seqs[i], list(range(2047, 2052)), f"sequence {i}")
    engine.close()


def test_sixty_four_unequal_prompts_then_single_tokens():
    from libllm_b200.engine import Engine
    folder, c, w = bench_model()
    g = torch.Generator().manual_seed(6)
    lens = torch.randint(300, 701, (64,), generator=g).tolist()
    lens[3], lens[40] = 300, 700
    seqs = [torch.randint(0, 128256, (n + 3,), generator=g).tolist() for n in lens]
    engine = Engine.from_folder(folder, dtype="bfloat16", max_tokens=sum((n + 3 + 63) // 64 * 64 for n in lens), max_seq_len=1024)
    got = run_prompts_then_single_tokens(engine, seqs, lens, 3)
    for i in (3, 40, 63):
        n = lens[i]
        check_rows_against_the_floor(got[i], c, w, seqs[i], list(range(n - 1, n + 3)), f"sequence {i} of length {n}")
    engine.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_same_two_batches_a_hundred_times_with_and_without_graphs(dtype):
    """Captured steps that take turns, slots and pages used again at once, kernels that start
    before their predecessors end: a hundred repetitions of two unequal batches must give, every
    time, what an engine that captures nothing gives (float32: the very same bits)."""
    from libllm_b200.engine import Engine
    name = "B"
    folder = model_folder(name)
    batches = [[("a", tokens_for(name, 40, 71), 33), ("b", tokens_for(name, 9, 72), 3), ("c", tokens_for(name, 70, 73), 64)],
               [("d", tokens_for(name, 21, 74), 20), ("e", tokens_for(name, 66, 75), 60)]]
    cap = max(sum((len(t) + 63) // 64 * 64 for _, t, _ in b) for b in batches)
    plain_engine = Engine.from_folder(folder, dtype=dtype, max_tokens=cap, use_graphs=False)
    want = [replay_batch(plain_engine, b) for b in batches]
    c, w = P.read_config(folder), plain_weights(folder)
    for b, res in zip(batches, want):
        for rid, toks, _ in b:
            check_logits(res[rid], P.forward_logits(c, w, toks), dtype, f"without graphs, {rid}")
    engine = Engine.from_folder(folder, dtype=dtype, max_tokens=cap)
    for rep in range(100):
        for b, res in zip(batches, want):
            got = replay_batch(engine, b)
            for rid, _, _ in b:
                if dtype == "float32":
                    assert torch.equal(got[rid], res[rid]), f"repetition {rep}, request {rid}: the bits differ"
                else:
                    # bfloat16: the graph's bound on the length shapes the key splits, so sums may be
                    # cut elsewhere; the distance to the other engine stays a rounding
                    assert rel_err(got[rid], res[rid].double()) < 2e-2, f"repetition {rep}, request {rid}"
    assert engine.info()["graph_replays"] > 1000
    assert engine.pages_in_use() == [0]
