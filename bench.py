#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on one GPU, as one JSON line.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

Default run: the layer sizes of Llama-3.2-1B with random bfloat16 weights, a batch of 8
sequences with 2,048-token prompts in a 4,096-token context; a "step" is one decode
step of the whole batch.  ``value`` is decoded tokens a second with the step timed on the
device (CUDA events on the engine's stream around K decode steps); ``e2e`` is the same through the Python entry
point (``Model.generate``), host token ids in and sampled ids out at every step.  The line
also carries the prefill of 2,048 tokens, the decode step's bytes against the memory
bandwidth, and decode at batch 1 and 64.  The decode step reads about 3 GB (weights and
cache), far more than the 126 MB L2, so no flush is needed between steps.
Only one GPU is supported: for --gpus N > 1 it says so and exits with 2."""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

LLAMA_1B = dict(model_type="llama", num_hidden_layers=16, hidden_size=2048, num_attention_heads=32,
                num_key_value_heads=8, head_dim=64, intermediate_size=8192, vocab_size=128256,
                rope_theta=500000.0,
                rope_scaling=dict(rope_type="llama3", factor=32.0, low_freq_factor=1.0, high_freq_factor=4.0,
                                  original_max_position_embeddings=8192),
                rms_norm_eps=1e-5, tie_word_embeddings=True, max_position_embeddings=131072,
                hidden_act="silu")
LLAMA_3B = dict(LLAMA_1B, num_hidden_layers=28, hidden_size=3072, num_attention_heads=24, num_key_value_heads=8,
                head_dim=128, intermediate_size=8192)
LLAMA_8B = dict(LLAMA_1B, num_hidden_layers=32, hidden_size=4096, num_attention_heads=32, num_key_value_heads=8,
                head_dim=128, intermediate_size=14336, tie_word_embeddings=False,
                rope_scaling=dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                                  original_max_position_embeddings=8192))
CONTEXT = 4096
PROMPT = 2048
FALLBACK_PEAKS = dict(hbm_gbs=6650.0, bf16_tflops=1590.0)


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        with open(path) as f:
            p = json.load(f)
        return dict(hbm_gbs=float(p["hbm_gbs"]), bf16_tflops=float(p["bf16_tflops"]), source="measured")
    return dict(FALLBACK_PEAKS, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows, self.proc = [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def stop(self):
        if self.proc is None:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["nvidia-smi unavailable"])
        self.proc.terminate()
        self.thread.join(timeout=2)
        sm = [float(r[0]) for r in self.rows if len(r) >= 6 and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in self.rows if len(r) >= 6 and r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({names[i] for r in self.rows if len(r) >= 6 for i in range(4) if r[2 + i] == "Active"})
        # "under load": a run also spends time where the GPU idles at a few hundred MHz (a model file
        # being written, a process starting); those samples say nothing about the timed kernels
        busy = [x for x in sm if x >= 0.5 * max(sm)] if sm else []
        return dict(sm_mhz=statistics.median(busy) if busy else None, sm_max_mhz=max(mx) if mx else None,
                    reasons=reasons, samples=len(sm), samples_under_load=len(busy))


def model_numbers(c):
    """Bytes a decode step has to read per weight pass and per cached token; prefill flops."""
    H, L, I, V = c["hidden_size"], c["num_hidden_layers"], c["intermediate_size"], c["vocab_size"]
    nH, nKV, d = c["num_attention_heads"], c["num_key_value_heads"], c["head_dim"]
    per_layer = H * (nH + 2 * nKV) * d + nH * d * H + 3 * H * I + 2 * H
    weight_bytes = 2 * (L * per_layer + V * H + H)          # every weight used once, the output matrix included
    kv_bytes_per_token = 2 * L * nKV * d * 2

    def prefill_flops(T, rows=1):
        # what the step has to compute: the last layer's feed-forward and the output matrix only for
        # the rows whose logits are wanted (the engine does no more, so no more is counted)
        lin = 2 * T * L * (H * (nH + 2 * nKV) * d + nH * d * H) + 2 * (T * (L - 1) + rows) * 3 * H * I
        att = L * 4 * nH * d * T * (T + 1) // 2            # q k^T and p v over the causal half
        return lin + att + 2 * rows * V * H
    return weight_bytes, kv_bytes_per_token, prefill_flops


LAST_STEP_TIMES = []          # milliseconds of each timed step of the last decode_rate call


def products_alone(cfg, tokens, pk):
    """The step's dominant kernel by itself: the tcgen05 products of a whole step (every layer's four,
    each layer with weights of its own so that none is met in L2, then the output matrix) launched one
    behind the other as in the step (one CUDA graph), without the attention and the norms between them: bytes of weights
    over time against the measured bandwidth.  What the step loses beyond this is the other kernels
    and the hand-overs to and from them."""
    import torch
    from libllm_b200.csrc import ops
    H, I, V, L = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"], cfg["num_hidden_layers"]
    nH, nKV, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    bf = torch.bfloat16
    shapes = [((nH + 2 * nKV) * d, H, False), (H, nH * d, False), (2 * I, H, True), (H, I, False)]
    jobs, nbytes = [], 0.0
    for layer in range(L + 1):
        for n, k, sw in (shapes if layer < L else [(V, H, False)]):
            x = torch.randn(tokens, k, device="cuda").to(bf)
            w = torch.empty(n, k, device="cuda", dtype=bf).normal_(0.0, 0.02)
            n_out = n // 2 if sw else n
            parts = 1 if sw or n == V else ops.gemm_tc_suggest_parts(tokens, n, k)
            out = torch.empty((tokens, n_out) if parts == 1 else (parts, tokens, n_out), dtype=bf if sw else torch.float32, device="cuda")
            jobs.append((x, w, out, sw))
            nbytes += 2.0 * n * k
    def run():
        for x, w, out, sw in jobs:
            ops.gemm_tc(x, w, out, swiglu=sw)
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        run()                                    # outside capture once: attributes, tensor maps
        side.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            run()
        times = []
        for rep in range(6):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(side)
            graph.replay()
            b.record(side)
            b.synchronize()
            if rep >= 2:
                times.append(a.elapsed_time(b) * 1e3)
    us = statistics.median(times)
    gbs = nbytes / (us * 1e-6) / 1e9
    return {"kernel": "gemm_tc_kernel: the step's products one behind the other, nothing between them",
            "launches": len(jobs), "us_per_step": round(us, 1), "gb_s": round(gbs, 1), "frac": round(gbs / pk["hbm_gbs"], 4)}


def decode_rate(model, batch, steps, warmup, vocab, seed=0):
    """Decoded tokens a second at ``batch`` with the steps timed on the device: CUDA events on the
    engine's stream around ``steps`` decode steps that are queued one behind the other (each takes
    its tokens from the one before on the device, so nothing waits for the host; the host queues a
    step in a small part of the time the device takes to run one).  Also returns the kernel
    launches of one step, counted by the host library while the step's graph was made."""
    import torch
    from libllm_b200 import _lib
    from libllm_b200.engine import GREEDY, StepItem
    eng = model.engine
    stream = torch.cuda.ExternalStream(eng.stream)
    g = torch.Generator().manual_seed(seed)
    slots = [eng.open_sequence() for _ in range(batch)]
    try:
        prompts = torch.randint(0, vocab, (batch, PROMPT), generator=g).tolist()
        # prompts in one step (the engine cuts it into launches of max_step_tokens)
        eng.step_tokens([StepItem(s, p, [PROMPT - 1]) for s, p in zip(slots, prompts)], GREEDY).result()
        fed = [StepItem(s, [0], [0], fed_row=i) for i, s in enumerate(slots)]
        n0 = _lib.lib().llm_kernel_launches()
        eng.step_tokens(fed, GREEDY).result()          # a shape's first step runs once and is captured once
        launches = (_lib.lib().llm_kernel_launches() - n0) // 2
        for _ in range(max(warmup - 1, 2)):
            eng.step_tokens(fed, GREEDY).result()
        marks = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
        eng.synchronize()
        marks[0].record(stream)
        pending = []
        for i in range(steps):
            pending.append(eng.step_tokens(fed, GREEDY))
            marks[i + 1].record(stream)
        for p in pending:
            p.result()
        eng.synchronize()
        ms = marks[0].elapsed_time(marks[steps]) / steps          # the K steps as one stretch: the record's figure
        LAST_STEP_TIMES[:] = [marks[i].elapsed_time(marks[i + 1]) for i in range(steps)]
        ctx_len = eng.sequence_length(slots[0])
        return batch * 1000.0 / ms, ms, ctx_len, launches
    finally:
        for s in slots:
            eng.close_sequence(s)


def e2e_rate(model, batch, steps, warmup, vocab, seed=1):
    """Decoded tokens a second through Model.generate, the call a user makes: token ids go in as
    Python lists and come out as Python lists.  Every step copies its descriptor (positions, page
    tables, token sources) from pinned host memory to the device and reads the sampled ids back;
    the clock is the host's, stamped when a step's tokens have arrived."""
    import torch
    g = torch.Generator().manual_seed(seed)
    prompts = torch.randint(0, vocab, (batch, PROMPT), generator=g).tolist()
    stamps = []

    def on_token(i, tok):
        if i == 0:
            stamps.append(time.perf_counter())

    model.generate(prompts, max_new_tokens=warmup + steps + 1, temperature=0.0, top_k=1, top_p=1.0, seed=0,
                   stop_token_ids=[], max_batch=batch, on_token=on_token)
    # stamps[0] follows the prompt step; steps warmup+1 .. warmup+steps are timed
    t = stamps[warmup + steps] - stamps[warmup]
    info = model.engine.info()
    return batch * steps / t, info["last_step_h2d_bytes"], info["last_step_d2h_bytes"]


def prefill_rate(model, vocab, flops_fn, peak_tflops, reps=3):
    import torch
    from libllm_b200.engine import StepItem
    eng = model.engine
    stream = torch.cuda.ExternalStream(eng.stream)
    g = torch.Generator().manual_seed(7)
    prompt = torch.randint(0, vocab, (PROMPT,), generator=g).tolist()
    times = []
    for r in range(reps + 2):
        s = eng.open_sequence()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        eng.synchronize()
        a.record(stream)
        eng.step([StepItem(s, prompt, [PROMPT - 1])])      # returns when the wanted row's logits are in host memory
        b.record(stream)
        eng.synchronize()
        eng.close_sequence(s)
        if r >= 2:
            times.append(a.elapsed_time(b))
    ms = statistics.median(times)
    flops = flops_fn(PROMPT)
    return dict(value=PROMPT * 1000.0 / ms, tokens=PROMPT, ms=ms, frac=flops / (ms * 1e-3) / (peak_tflops * 1e12))


def run_workload(args):
    """The two larger workloads the benchmark description names, through Model.generate (host token ids in
    and out): Llama-3.2-3B sizes with 16 prompts of lengths uniform in [128, 2048] and 256 decoded tokens
    each; Llama-3.1-8B sizes with 32 prompts of 4,096 tokens and 512 decoded tokens each.  One JSON line:
    time to the first tokens (all prompts in one step), decoded tokens a second after it, and the bytes
    the decode steps had to read against the memory bandwidth."""
    import torch
    from libllm_b200 import Model
    if args.workload == "3b":
        cfg, n_new = dict(LLAMA_3B), 256
        g = torch.Generator().manual_seed(11)
        lens = torch.randint(128, 2049, (16,), generator=g).tolist()
        context = 2048 + n_new
    else:
        cfg, n_new = dict(LLAMA_8B), 512
        lens = [4096] * 32
        context = 8192
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    g = torch.Generator().manual_seed(12)
    prompts = [torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist() for n in lens]
    pages = sum((n + n_new + 63) // 64 for n in lens)
    model = Model.from_random(cfg, seed=0, dtype="bfloat16", max_tokens=pages * 64, max_seq_len=context)
    stamps = []

    def on_token(i, tok):
        if i == 0:
            stamps.append(time.perf_counter())

    model.generate(prompts[:2], max_new_tokens=4, temperature=0.0, stop_token_ids=[])        # kernels loaded, graphs not
    t0 = time.perf_counter()
    out = model.generate(prompts, max_new_tokens=n_new, temperature=0.0, stop_token_ids=[], max_batch=len(prompts),
                         on_token=on_token)
    t1 = time.perf_counter()
    assert all(len(o) == n_new for o in out)
    wbytes, kv_per_tok, flops_fn = model_numbers(cfg)
    pk = peaks()
    ttft = stamps[0] - t0
    decode_s = t1 - stamps[0]
    steps = n_new - 1
    mean_ctx = sum(lens) / len(lens) + n_new / 2
    step_bytes = wbytes + len(lens) * mean_ctx * kv_per_tok
    prefill_flops = sum(flops_fn(n) for n in lens)
    print(json.dumps({
        "workload": args.workload, "impl": "ours", "dtype": "bf16", "data": "synthetic",
        "config": {"layers": cfg["num_hidden_layers"], "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"],
                   "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
                   "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"], "batch": len(lens),
                   "prompt_tokens": sum(lens), "new_tokens_each": n_new},
        "prefill": {"tokens": sum(lens), "ms": round(ttft * 1e3, 2), "tok_s": round(sum(lens) / ttft, 1),
                    "frac": round(prefill_flops / ttft / (pk["bf16_tflops"] * 1e12), 4)},
        "decode": {"tok_s": round(len(lens) * steps / decode_s, 1), "ms_per_step": round(decode_s / steps * 1e3, 3),
                   "hbm_frac": round(step_bytes / (decode_s / steps) / 1e9 / pk["hbm_gbs"], 4)},
        "total_s": round(t1 - t0, 3)}))
    return 0


def run_reference(args):
    """The reference arm: ling0322/libllm's unmodified C++/CUDA code (compiled into baseline/_ref by
    baseline/reference_arm.py; it has no installable Python package of its engine) at the same layer
    sizes, batch and prompt length, in its own compute type (float16), timed with a device
    synchronisation on both sides.  Where it cannot be built or run, one line says why."""
    def unavailable(why):
        print(json.dumps({"impl": "reference", "unavailable": " ".join(str(why).split())[:600]}))
        return 0
    if args.gpus != 1:
        return unavailable("ling0322/libllm runs on one GPU (every CUDA call of it targets device 0)")
    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    try:
        import reference_arm
        reference_arm.build()
    except Exception as e:                       # no checkout, no compiler, a compile error
        return unavailable(f"the reference could not be compiled here: {e}")
    try:
        import torch
        if not torch.cuda.is_available():
            return unavailable("no CUDA device")
    except ImportError:
        pass
    cfg = dict(LLAMA_1B)
    full_layers = cfg["num_hidden_layers"]
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    warmup = max(args.warmup, 3)
    sampler = ClockSampler()
    sampler.start()
    try:
        r = reference_arm.run(cfg, PROMPT, args.batch, args.steps, warmup, CONTEXT)
    except Exception as e:
        sampler.stop()
        return unavailable(f"the reference's driver failed: {e}")
    clocks = sampler.stop()
    pk = peaks()
    wbytes, kv_per_tok, flops_fn = model_numbers(cfg)
    ms, e2e_ms = r["decode_ms_per_step"], r["e2e_ms_per_step"]
    step_bytes = wbytes + args.batch * (PROMPT + warmup + args.steps // 2) * kv_per_tok
    achieved = step_bytes / (ms * 1e-3) / 1e9
    print(json.dumps({
        "metric": "decode tok/s (Llama-3.2-1B layer sizes, batch 8, 2048-token prompts, 4096 context)",
        "value": round(args.batch * 1000.0 / ms, 1), "unit": "tok/s", "n_gpus": 1, "steps": args.steps, "warmup": warmup,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "fp16", "data": "synthetic", "impl": "reference",
        "config": {"model": "llama-3.2-1b-sizes", "layers": cfg["num_hidden_layers"], "layers_full": full_layers,
                   "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
                   "head_dim": cfg["head_dim"], "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"],
                   "global_batch": args.batch, "seq_len": CONTEXT, "prompt_len": PROMPT, "parallelism": "single-gpu",
                   "weights": "random fp16 N(0,0.02), tied", "attention": "the reference's portable path (FlashAttention off)",
                   "l2": "step reads more than L2 (no flush)", "peaks": pk["source"]},
        "e2e": {"value": round(args.batch * 1000.0 / e2e_ms, 1), "unit": "tok/s", "h2d_bytes_per_step": 8 * args.batch,
                "d2h_bytes_per_step": 8 * args.batch},
        "clocks": clocks,
        "prefill": {"value": round(PROMPT * 1000.0 / r["prefill_ms"], 1), "tokens": PROMPT, "ms": round(r["prefill_ms"], 4),
                    "frac": round(flops_fn(PROMPT) / (r["prefill_ms"] * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)}}))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the configuration (named in config)")
    ap.add_argument("--no-points", action="store_true", help="skip decode at batch 1 and 64")
    ap.add_argument("--workload", choices=["1b", "3b", "8b"], default="1b",
                    help="1b: the benchmark line (default); 3b, 8b: the larger workloads, a line of their own")
    ap.add_argument("--only", choices=["decode", "prefill"], default=None,
                    help="run one part only and print a short line (for profiling; not a bench record)")
    ap.add_argument("--prompt-len", type=int, default=None,
                    help="with --only: prompts of this many tokens instead of 2048 (the context grows to fit)")
    args = ap.parse_args()
    if args.prompt_len:
        if not args.only:
            print("bench.py: --prompt-len goes with --only (the record is taken at the sizes BASELINE.json names)")
            return 2
        global PROMPT, CONTEXT
        PROMPT = args.prompt_len
        CONTEXT = max(CONTEXT, PROMPT + 2048)
    if args.impl == "reference":
        return run_reference(args)
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    args.warmup = max(args.warmup, 3)
    if args.workload != "1b":
        return run_workload(args)

    import torch
    from libllm_b200 import Model
    cfg = dict(LLAMA_1B)
    full_layers = cfg["num_hidden_layers"]
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    pk = peaks()
    wbytes, kv_per_tok, flops_fn = model_numbers(cfg)
    vocab = cfg["vocab_size"]
    max_batch = max(args.batch, 1 if (args.no_points or args.only) else 64)
    model = Model.from_random(cfg, seed=0, dtype="bfloat16", max_tokens=max_batch * CONTEXT, max_seq_len=CONTEXT)

    if args.only == "decode":
        rate, ms, ctx_len, _ = decode_rate(model, args.batch, args.steps, args.warmup, vocab)
        step_bytes = wbytes + args.batch * ctx_len * kv_per_tok
        print(json.dumps({"only": "decode", "batch": args.batch, "tok_s": round(rate, 1), "ms_per_step": round(ms, 4),
                          "context": ctx_len, "hbm_frac": round(step_bytes / (ms * 1e-3) / 1e9 / pk["hbm_gbs"], 4)}))
        return 0
    if args.only == "prefill":
        print(json.dumps({"only": "prefill", **prefill_rate(model, vocab, flops_fn, pk["bf16_tflops"])}))
        return 0
    sampler = ClockSampler()
    sampler.start()
    rate, ms, ctx_len, launches_per_step = decode_rate(model, args.batch, args.steps, args.warmup, vocab)
    clocks = sampler.stop()
    step_times = sorted(LAST_STEP_TIMES)
    median_ms = step_times[len(step_times) // 2] if step_times else ms
    e2e, h2d, d2h = e2e_rate(model, args.batch, args.steps, args.warmup, vocab)
    prefill = prefill_rate(model, vocab, flops_fn, pk["bf16_tflops"])
    step_bytes = wbytes + args.batch * ctx_len * kv_per_tok
    achieved = step_bytes / (ms * 1e-3) / 1e9
    points = {}
    if not args.no_points:
        for b in (1, 64):
            r, _, _, _ = decode_rate(model, b, max(8, args.steps // 2), args.warmup, vocab)
            points[f"decode_b{b}"] = round(r, 1)
    line = {
        "metric": "decode tok/s (Llama-3.2-1B layer sizes, batch 8, 2048-token prompts, 4096 context)",
        "value": round(rate, 1), "unit": "tok/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms, 4), "ms_per_step_median": round(median_ms, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": "ours",
        "config": {"model": "llama-3.2-1b-sizes", "layers": cfg["num_hidden_layers"], "layers_full": full_layers,
                   "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"],
                   "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
                   "intermediate": cfg["intermediate_size"], "vocab": vocab, "global_batch": args.batch,
                   "seq_len": CONTEXT, "prompt_len": PROMPT, "context_at_timing": ctx_len,
                   "parallelism": "single-gpu", "weights": "random bf16 N(0,0.02), tied",
                   "l2": "step reads more than L2 (no flush)", "peaks": pk["source"]},
        "e2e": {"value": round(e2e, 1), "unit": "tok/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": launches_per_step * args.steps,
        "clocks": clocks,
        "prefill": {k: (round(v, 4) if isinstance(v, float) else v) for k, v in prefill.items()},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points,
        "dominant_kernel": products_alone(cfg, args.batch, pk),
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
