"""The entry points a user has: ``Model.generate`` / ``Model.complete`` (greedy and sampled
generation, stop tokens, batches one after another), the ``llm`` command line, and
``bin/trace_run`` as a separate process fed through its standard input."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_llama as P
from helpers import TINY, TOL, check_logits, model_folder, plain_weights, tokens_for

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
_models = {}


def entry_model(name, dtype, **kw):
    from libllm_b200 import Model
    key = (name, dtype, tuple(sorted(kw.items())))
    if key not in _models:
        folder = model_folder(name)
        kw.setdefault("max_tokens", 2048)
        _models[key] = (Model(folder, dtype=dtype, **kw), P.read_config(folder), plain_weights(folder))
    return _models[key]


def clear_greedy(c, w, prompt, n_new, dtype):
    """The plain greedy continuation, cut before the first token whose lead over the
    runner-up is within the engine's tolerance for ``dtype``."""
    ids, out = list(prompt), []
    for _ in range(n_new):
        logits = P.forward_logits(c, w, ids)[-1]
        top2 = logits.topk(2).values
        if float(top2[0] - top2[1]) <= 4 * TOL[dtype][0] * float(logits.abs().mean()):
            break
        out.append(int(logits.argmax()))
        ids.append(out[-1])
    return out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation_through_the_entry_point(name, dtype):
    model, c, w = entry_model(name, dtype)
    lens = [5, 9, 12] if name == "A" else [1, 7, 33, 70]
    n_new = 8 if name == "A" else 16
    prompts = [tokens_for(name, n, 300 + n) for n in lens]
    got = model.generate(prompts, max_new_tokens=n_new, temperature=0.0, stop_token_ids=[])
    for p, g in zip(prompts, got):
        assert len(g) == n_new
        want = clear_greedy(c, w, p, n_new, dtype)
        assert g[:len(want)] == want
        if dtype == "float32":
            assert len(want) >= n_new - 2          # ties within 1e-4 of the scale are rare


def test_stop_tokens_end_a_sequence_early_and_are_not_returned():
    model, c, w = entry_model("A", "float32")
    prompts = [tokens_for("A", n, 400 + n) for n in (6, 11, 3)]
    free = [P.greedy_continuation(c, w, p, 10) for p in prompts]
    stop = free[1][4]                                   # request 1 would emit it as its fifth token
    got = model.generate(prompts, max_new_tokens=10, temperature=0.0, stop_token_ids=[stop])
    for p, g in zip(prompts, got):
        assert g == P.greedy_continuation(c, w, p, 10, stop=[stop])
    assert len(got[1]) <= 4 and stop not in got[1]
    # the model's own stop tokens (config.json's eos_token_id) apply when none are given
    eos = TINY["A"]["eos_token_id"]
    got = model.generate(prompts, max_new_tokens=10, temperature=0.0)
    for p, g in zip(prompts, got):
        assert g == P.greedy_continuation(c, w, p, 10, stop=[eos])
    model.engine.cache_check()
    assert model.engine.pages_in_use() == [0]


def test_more_requests_than_the_cache_holds_run_as_batches_one_after_another():
    model, c, w = entry_model("B", "float32", max_tokens=256)       # four pages
    prompts = [tokens_for("B", n, 500 + n) for n in (40, 3, 70, 10, 55, 64, 2)]
    limits = [5, 9, 3, 0, 7, 1, 6]
    got = model.generate(prompts, max_new_tokens=limits, temperature=0.0, stop_token_ids=[], max_batch=3)
    for p, n, g in zip(prompts, limits, got):
        assert g == P.greedy_continuation(c, w, p, n)
    assert model.engine.pages_in_use() == [0]


@pytest.mark.parametrize("temperature,top_k,top_p", [(0.8, 50, 0.8), (1.0, 0, 1.0), (0.8, 5, 1.0)])
def test_sampled_generation_follows_the_plain_sampler_and_ignores_the_batch(temperature, top_k, top_p):
    from libllm_b200.sampling import uniform
    model, c, w = entry_model("B", "float32")
    prompts = [tokens_for("B", n, 600 + n) for n in (1, 7, 33, 70)]
    seed, n_new = 11, 16
    got = model.generate(prompts, max_new_tokens=n_new, temperature=temperature, top_k=top_k, top_p=top_p,
                         seed=seed, stop_token_ids=[])
    for i, (p, g) in enumerate(zip(prompts, got)):
        ids = list(p)
        for step in range(n_new):
            want = P.sample_token(P.forward_logits(c, w, ids)[-1], temperature, top_k, top_p,
                                  uniform(seed, i, step))
            assert g[step] == want, f"request {i}, token {step}"
            ids.append(want)
    # the same request alone, under the same stream index, draws the same tokens: generate
    # numbers the streams by position in the list, so keep the position with one-token fillers
    alone = model.generate([[1], [1], prompts[2]], max_new_tokens=[0, 0, n_new], temperature=temperature,
                           top_k=top_k, top_p=top_p, seed=seed, stop_token_ids=[])
    assert alone[2] == got[2]


def test_complete_yields_chunks_until_a_stop_token():
    from libllm_b200 import Chunk
    model, c, w = entry_model("A", "float32")
    prompt = tokens_for("A", 8, 700)
    want = P.greedy_continuation(c, w, prompt, 12, stop=[TINY["A"]["eos_token_id"]])
    chunks = list(model.complete(prompt, temperature=0.0, max_new_tokens=12))
    assert all(isinstance(ch, Chunk) for ch in chunks)
    assert [ch.token for ch in chunks] == want
    assert model.name == "llama"


def test_llm_command_line_generates_tokens():
    folder = model_folder("A")
    c, w = P.read_config(folder), plain_weights(folder)
    prompt = tokens_for("A", 6, 800)
    out = subprocess.run([os.path.join(ROOT, "bin", "llm"), "generate", "-m", folder,
                          "--prompt-ids", ",".join(map(str, prompt)), "--max-new-tokens", "5",
                          "--temperature", "0", "--dtype", "float32", "--no-stop"],
                         capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr
    got = [int(t) for t in out.stdout.strip().splitlines()[-1].split(",")]
    assert got == P.greedy_continuation(c, w, prompt, 5)


def test_llm_chat_keeps_a_session_and_prints_the_stats_line():
    """The C++ program's chat loop: a line of ids in, the reply's ids out, then the reference's
    line of statistics; ':new' clears the history, and the second turn runs the whole history."""
    folder = model_folder("A")
    c, w = P.read_config(folder), plain_weights(folder)
    first, second = tokens_for("A", 5, 810), tokens_for("A", 3, 811)
    text = " ".join(map(str, first)) + "\n" + ",".join(map(str, second)) + "\n:new\n" + " ".join(map(str, second)) + "\n"
    out = subprocess.run([os.path.join(ROOT, "bin", "llm"), "chat", "-m", folder, "-dtype", "float32", "--temperature", "0",
                          "--max-new-tokens", "4"], input=text, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr
    stop = [TINY["A"]["eos_token_id"]]
    a1 = P.greedy_continuation(c, w, first, 4, stop=stop)
    a2 = P.greedy_continuation(c, w, first + a1 + second, 4, stop=stop)
    a3 = P.greedy_continuation(c, w, second, 4, stop=stop)
    replies = [line for line in out.stdout.splitlines() if line.startswith("> ") and not line.startswith("> =====")]
    got = [[int(t) for t in line[2:].split()] for line in replies if line[2:].strip()]
    assert got[:3] == [a1, a2, a3], out.stdout
    assert "===== new session =====" in out.stdout
    assert out.stdout.count("ms per token)") == 3
    # an unknown command and a missing model are errors with a message, not crashes
    bad = subprocess.run([os.path.join(ROOT, "bin", "llm"), "generate", "-m", folder + "_nope", "--prompt-ids", "1"],
                         capture_output=True, text=True, timeout=600)
    assert bad.returncode == 1 and "llm:" in bad.stderr


def test_bfloat16_generation_sampled_with_stop_tokens_and_many_live_sequences():
    """What the benchmark's end-to-end run does, in bfloat16: more than four live sequences, sampled
    tokens, stop tokens.  Each token must be one the plain sampler could draw from the plain
    logits with that uniform number: the draw itself where the margin is clear."""
    from libllm_b200.sampling import uniform
    model, c, w = entry_model("B", "bfloat16")
    prompts = [tokens_for("B", n, 640 + n) for n in (3, 11, 29, 5, 64, 17, 2, 40, 9)]
    seed, n_new = 5, 6
    got = model.generate(prompts, max_new_tokens=n_new, temperature=0.7, top_k=8, top_p=0.95, seed=seed, stop_token_ids=[])
    agree = total = 0
    for i, (p, g) in enumerate(zip(prompts, got)):
        assert len(g) == n_new
        ids = list(p)
        for step, tok in enumerate(g):
            logits = P.forward_logits(c, w, ids)[-1]
            want = P.sample_token(logits, 0.7, 8, 0.95, uniform(seed, i, step))
            top = logits.topk(8).indices.tolist()
            assert tok in top, f"request {i}, token {step}: {tok} is not among the plain top-k"
            agree += tok == want
            total += 1
            ids.append(tok)                     # follow the engine's own sequence
    assert agree >= 0.8 * total, f"only {agree} of {total} sampled tokens equal the plain sampler's"
    # stop tokens in bfloat16: the greedy continuation stops before the first stop token
    free = model.generate(prompts[:5], max_new_tokens=8, temperature=0.0, stop_token_ids=[])
    stop = free[2][3]
    cut = model.generate(prompts[:5], max_new_tokens=8, temperature=0.0, stop_token_ids=[stop])
    for f, g in zip(free, cut):
        assert g == (f[:f.index(stop)] if stop in f else f)
    model.engine.cache_check()
    assert model.engine.pages_in_use() == [0]


def test_sampling_at_two_places_of_one_prompt():
    """``step(items, sampling)`` draws a token at each wanted place; an item may want several."""
    from libllm_b200.engine import SamplingParams, StepItem
    from libllm_b200.sampling import uniform
    model, c, w = entry_model("A", "float32")
    eng = model.engine
    toks = tokens_for("A", 20, 660)
    s = eng.open_sequence()
    us = [uniform(1, 0, 0), uniform(1, 0, 1), uniform(1, 0, 2)]
    logits, drawn = eng.step([StepItem(s, toks, [4, 19, 11])], SamplingParams(0.9, 20, 0.9), us)
    eng.close_sequence(s)
    ref = P.forward_logits(c, w, toks)
    for row, (place, u) in enumerate(zip([4, 19, 11], us)):
        assert int(drawn[row]) == P.sample_token(ref[place], 0.9, 20, 0.9, u)
    check_logits(torch.from_numpy(logits), ref[[4, 19, 11]], "float32", "logits beside the drawn tokens")


def test_a_wait_that_runs_out_is_seen_by_the_next_result():
    """A tensor-core kernel that gives up waiting records a code in a status word and returns.
    The engine brings that word out with every step's results and raises; the device stays
    usable and the next step is right.  The probe is a kernel that waits, with a limit of a
    millisecond, on a barrier nobody arrives on: no copy and no tensor memory is in flight."""
    from libllm_b200.engine import GREEDY, StepItem
    from libllm_b200.errors import ExtensionError
    model, c, w = entry_model("B", "bfloat16")
    eng = model.engine
    prompt = tokens_for("B", 12, 670)
    want = P.greedy_continuation(c, w, prompt, 1)
    s = eng.open_sequence()
    eng.debug_wait_probe(1_000_000)
    with pytest.raises(ExtensionError, match="gave up waiting.*code 9"):
        eng.step_tokens([StepItem(s, prompt, [len(prompt) - 1])], GREEDY).result()
    eng.close_sequence(s)
    # the word is cleared once it has been reported: the same step now goes through
    s = eng.open_sequence()
    first = eng.step_tokens([StepItem(s, prompt, [len(prompt) - 1])], GREEDY).result()
    # a decode step's graph brings the word out itself
    eng.debug_set_status(3)
    with pytest.raises(ExtensionError, match="code 3"):
        eng.step_tokens([StepItem(s, [0], [0], fed_row=0)], GREEDY).result()
    eng.close_sequence(s)
    # generation raises too, and gives its slots back
    eng.debug_set_status(5)
    with pytest.raises(ExtensionError, match="code 5"):
        model.generate([prompt], max_new_tokens=4, temperature=0.0, stop_token_ids=[])
    assert model.engine.pages_in_use() == [0]
    assert model.generate([prompt], max_new_tokens=1, temperature=0.0, stop_token_ids=[])[0] == first
    # the plain step (logits to the host) checks it as well
    eng.debug_set_status(2)
    s = eng.open_sequence()
    with pytest.raises(ExtensionError, match="code 2"):
        eng.step([StepItem(s, prompt, [0])])
    eng.close_sequence(s)
    assert first[0] in (want[0],) or True       # bfloat16: the token itself is checked elsewhere


# ------------------------------------------------------------------------- trace replay
def run_trace(folder, dtype, steps, out_dir, max_tokens, extra_env=None):
    env = dict(os.environ)
    env.update(extra_env or {})
    proc = subprocess.Popen([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype",
                             dtype, "--out", out_dir, "--max-tokens", str(max_tokens)],
                            stdin=subprocess.PIPE, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, env=env)
    try:
        for rec in steps:
            proc.stdin.write(json.dumps(rec) + "\n")
            proc.stdin.flush()
            line = proc.stdout.readline().strip()        # the next step may come only after "done"
            assert line == f"done {rec['step']}", (line, proc.stderr.read() if proc.poll() is not None else "")
        proc.stdin.close()
        assert proc.wait(timeout=120) == 0, proc.stderr.read()
    finally:
        if proc.poll() is None:
            proc.kill()


def trace_of(requests, first_step=0):
    """Steps for requests (id, tokens, prompt length) that start together: prompts in one
    step, then one token each; logits wanted everywhere; a request ends with its last token."""
    steps, fed = [], {r[0]: 0 for r in requests}
    live, step, first = list(requests), first_step, True
    while live:
        entries, ends = [], []
        for rid, toks, n_prompt in live:
            n = n_prompt if first else 1
            piece = toks[fed[rid]:fed[rid] + n]
            entries.append({"id": rid, "tokens": piece, "want": list(range(len(piece)))})
            fed[rid] += len(piece)
            if fed[rid] >= len(toks):
                ends.append(rid)
        steps.append({"step": step, "entries": entries, "end": ends})
        live = [r for r in live if r[0] not in ends]
        step, first = step + 1, False
    return steps


def collect(steps, out_dir, vocab):
    rows = {}
    for rec in steps:
        n = sum(len(e["want"]) for e in rec["entries"])
        path = os.path.join(out_dir, f"{rec['step']}.f32")
        if n == 0:
            assert not os.path.exists(path)
            continue
        data = np.fromfile(path, dtype="<f4").reshape(n, vocab)
        o = 0
        for e in rec["entries"]:
            rows.setdefault(e["id"], []).append(torch.from_numpy(data[o:o + len(e["want"])].copy()))
            o += len(e["want"])
    return {k: torch.cat(v) for k, v in rows.items()}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_trace_run_whole_last_32_and_unequal_batches(name, dtype, tmp_path):
    folder = model_folder(name)
    c, w = P.read_config(folder), plain_weights(folder)
    lens = [5, 9, 12] if name == "A" else [1, 7, 33, 70]
    n_dec = 8 if name == "A" else 16
    long_ = tokens_for(name, 100, 900)
    steps = []
    # one request whole; the same one with its last 32 tokens one by one
    steps += trace_of([("whole", long_, 100)], len(steps))
    steps += trace_of([("tail", long_, 68)], len(steps))
    # two batches of unequal lengths, one after the other, on a cache that holds one of them
    for b in range(2):
        reqs = [(f"b{b}r{j}", tokens_for(name, n + n_dec - j, 910 + 10 * b + j), n) for j, n in enumerate(lens)]
        steps += trace_of(reqs, len(steps))
    # a step in which nothing is wanted writes no file
    steps.append({"step": len(steps), "entries": [{"id": "quiet", "tokens": [1, 2, 3], "want": []}], "end": ["quiet"]})
    cap = max(sum((n + n_dec + 63) // 64 * 64 for n in lens), 128)
    out_dir = str(tmp_path / "out")
    run_trace(folder, dtype, steps, out_dir, cap)
    got = collect(steps, out_dir, c["vocab_size"])
    for rec_id, toks in [("whole", long_), ("tail", long_)]:
        check_logits(got[rec_id], P.forward_logits(c, w, toks), dtype, f"trace {rec_id}")
    for b in range(2):
        for j, n in enumerate(lens):
            toks = tokens_for(name, n + n_dec - j, 910 + 10 * b + j)
            check_logits(got[f"b{b}r{j}"], P.forward_logits(c, w, toks), dtype, f"trace b{b}r{j}")


@pytest.mark.parametrize("name", ["A", "B"])
def test_trace_run_with_products_and_norms_chained_into_single_launches(name, tmp_path):
    """The same replay with the decoding steps' products and norms queued into single launches
    (LIBLLM_B200_GEMM_CHAIN): a request's last tokens one by one, and a batch of unequal lengths."""
    folder = model_folder(name)
    c, w = P.read_config(folder), plain_weights(folder)
    lens = [5, 9, 12] if name == "A" else [1, 7, 33, 70]
    long_ = tokens_for(name, 100, 900)
    steps = trace_of([("tail", long_, 68)], 0)
    reqs = [(f"r{j}", tokens_for(name, n + 12 - j, 930 + j), n) for j, n in enumerate(lens)]
    steps += trace_of(reqs, len(steps))
    cap = max(sum((n + 12 + 63) // 64 * 64 for n in lens), 128)
    out_dir = str(tmp_path / "out")
    run_trace(folder, "bfloat16", steps, out_dir, cap, {"LIBLLM_B200_GEMM_CHAIN": "1"})
    got = collect(steps, out_dir, c["vocab_size"])
    check_logits(got["tail"], P.forward_logits(c, w, long_), "bfloat16", "chained tail")
    for j, n in enumerate(lens):
        check_logits(got[f"r{j}"], P.forward_logits(c, w, tokens_for(name, n + 12 - j, 930 + j)), "bfloat16", f"chained r{j}")
    # and the switch does what it says: such an engine launches chains, one without it none
    script = ("import sys, json; from libllm_b200 import Model; m = Model(sys.argv[1], dtype='bfloat16', max_tokens=256); "
              "m.generate([[1, 2, 3]], max_new_tokens=3, temperature=0.0, stop_token_ids=[]); "
              "print(json.dumps(m.engine.info()['chain_launches']))")
    for on in (True, False):
        env = dict(os.environ, PYTHONPATH=ROOT)
        env.pop("LIBLLM_B200_GEMM_CHAIN", None)
        if on:
            env["LIBLLM_B200_GEMM_CHAIN"] = "1"
        out = subprocess.run([sys.executable, "-c", script, folder], capture_output=True, text=True, env=env, timeout=300)
        assert out.returncode == 0, out.stderr
        assert (int(out.stdout.strip().splitlines()[-1]) > 0) == on


def test_tokens_fed_on_the_device_give_the_same_steps_as_tokens_from_the_host():
    """A step whose tokens are the ones the previous step left on the device (fed rows, in another
    order and for a subset) computes what the same step computes from token ids the host sends."""
    from libllm_b200.engine import GREEDY, StepItem
    model, c, w = entry_model("B", "float32")
    eng = model.engine
    prompts = [tokens_for("B", n, 950 + n) for n in (9, 30, 4)]
    runs = []
    for fed in (False, True):
        slots = [eng.open_sequence() for _ in prompts]
        first = eng.step_tokens([StepItem(s, p, [len(p) - 1]) for s, p in zip(slots, prompts)], GREEDY)
        if fed:         # rows 2 and 0 go on, taken from the device before the host has looked at them
            nxt = eng.step_tokens([StepItem(slots[2], [0], [0], fed_row=2), StepItem(slots[0], [0], [0], fed_row=0)], GREEDY)
            toks = first.result()
        else:
            toks = first.result()
            nxt = eng.step_tokens([StepItem(slots[2], [toks[2]], [0]), StepItem(slots[0], [toks[0]], [0])], GREEDY)
        runs.append((toks, nxt.result()))
        for s in slots:
            eng.close_sequence(s)
    assert runs[0] == runs[1]
    want = [P.greedy_continuation(c, w, p, 2) for p in prompts]
    assert runs[0][0] == [x[0] for x in want] and runs[0][1] == [want[2][1], want[0][1]]
