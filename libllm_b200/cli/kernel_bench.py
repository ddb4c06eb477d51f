"""Times one kernel of the library alone, at given sizes, against its roofline.

    python -m libllm_b200.cli.kernel_bench gemv --m 8 --n 128256 --k 2048
    python -m libllm_b200.cli.kernel_bench attention_decode --batch 64 --context 2048
    python -m libllm_b200.cli.kernel_bench attention_prefill --tokens 2048
    python -m libllm_b200.cli.kernel_bench layer_products --m 8      # the four products of one layer
    python -m libllm_b200.cli.kernel_bench chain_layer --m 8         # a layer's products and norms as one launch

One JSON line per run: microseconds per launch (CUDA events on the launching stream,
after warm-up, with a buffer larger than L2 written between launches), the bytes the
kernel has to move or the flops it has to do, and the fraction of the peak.  The
reference keeps such microbenchmarks for its operators at Llama-3.2-3B shapes
(src/flint/cuda/benchmark.cc:139-179); these are the ones its published tables list.

With ``--iters 1 --warmup 0`` the program launches the kernel once: that form is the one
to run under a profiler."""
from __future__ import annotations

import argparse
import json
import math
import os
import sys

L2_BYTES = 126 * 1024 * 1024
FALLBACK_PEAKS = dict(hbm_gbs=6650.0, bf16_tflops=1590.0)


def peaks():
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    path = os.path.join(root, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        with open(path) as f:
            p = json.load(f)
        return dict(hbm_gbs=float(p["hbm_gbs"]), bf16_tflops=float(p["bf16_tflops"]), source="measured")
    return dict(FALLBACK_PEAKS, source="fallback")


class Timer:
    def __init__(self, iters: int, warmup: int, flush: bool = True):
        import torch
        self.torch = torch
        self.iters, self.warmup = iters, warmup
        self.flusher = torch.empty(2 * L2_BYTES, dtype=torch.uint8, device="cuda") if flush else None

    def run(self, fn) -> float:
        """Median microseconds of one call of ``fn``."""
        torch = self.torch
        for _ in range(self.warmup):
            fn()
        times = []
        for _ in range(self.iters):
            if self.flusher is not None:
                self.flusher.fill_(1)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            b.synchronize()
            times.append(a.elapsed_time(b) * 1e3)
        times.sort()
        return times[len(times) // 2]


def report(name, us, bytes_moved=None, flops=None, **sizes):
    pk = peaks()
    line = dict(kernel=name, **sizes, us=round(us, 2), peaks=pk["source"])
    if bytes_moved is not None:
        gbs = bytes_moved / (us * 1e-6) / 1e9
        line.update(bytes=int(bytes_moved), gbs=round(gbs, 1), hbm_frac=round(gbs / pk["hbm_gbs"], 4))
    if flops is not None:
        tf = flops / (us * 1e-6) / 1e12
        line.update(flops=int(flops), tflops=round(tf, 2), bf16_frac=round(tf / pk["bf16_tflops"], 4))
    print(json.dumps(line), flush=True)
    return line


# ---------------------------------------------------------------------------------- kernels
def bench_gemv(args, timer, M=None, N=None, K=None, swiglu=None, name="gemv"):
    import torch
    from ..csrc import ops
    M, N, K = M or args.m, N or args.n, K or args.k
    swiglu = args.swiglu if swiglu is None else swiglu
    x = torch.randn(M, K, device="cuda").to(torch.bfloat16)
    w = (torch.randn(N, K, device="cuda") * 0.02).to(torch.bfloat16)
    out_dtype = torch.bfloat16 if swiglu else torch.float32

    def fn():
        if args.library:
            y = torch.mm(x, w.t()).float()
            if swiglu:
                ops.swiglu(y, torch.empty((M, N // 2), dtype=torch.bfloat16, device="cuda"))
            return
        if args.tc:
            n = N // 2 if swiglu else N
            parts = 1 if swiglu else ops.gemm_tc_suggest_parts(M, N, K)
            shape = (M, n) if parts == 1 else (parts, M, n)
            ops.gemm_tc(x, w, torch.empty(shape, dtype=out_dtype, device="cuda"), swiglu=swiglu)
            return
        assert ops.gemv_supported(x, w), "the mma.sync weight streamer refuses these sizes"
        n = N // 2 if swiglu else N
        parts = 1 if swiglu else ops.gemv_suggest_parts(M, N, K)
        shape = (M, n) if parts == 1 else (parts, M, n)
        ops.gemv_bf16(x, w, torch.empty(shape, dtype=out_dtype, device="cuda"), swiglu=swiglu)
    us = timer.run(fn)
    n_out = N // 2 if swiglu else N
    if args.library:
        name += " (library)"
    if args.tc:
        name += " (tcgen05)"
    return report(name, us, bytes_moved=2 * N * K + 2 * M * K + M * n_out * (2 if swiglu else 4),
                  flops=2 * M * N * K, m=M, n=N, k=K, swiglu=bool(swiglu))


def bench_layer_products(args, timer):
    """The four products of one Llama-3.2-1B-sized layer and the output matrix at --m tokens."""
    H, I, V = args.hidden, args.intermediate, args.vocab
    qkv = (args.heads + 2 * args.kv_heads) * args.head_dim
    total = 0.0
    for name, n, k, sw in (("qkv", qkv, H, False), ("o", H, args.heads * args.head_dim, False),
                           ("gate_up+swiglu", 2 * I, H, True), ("down", H, I, False), ("lm_head", V, H, False)):
        total += bench_gemv(args, timer, args.m, n, k, sw, name=name)["us"]
    print(json.dumps({"layer_products_us": round(total, 1)}))


def _paged_cache(B, ctx, n_kv, d, page=64, dtype=None):
    import torch
    dtype = dtype or torch.bfloat16
    per_seq = (ctx + page - 1) // page
    n_pages = B * per_seq
    k = (torch.randn(n_pages, n_kv, page, d, device="cuda") * 0.5).to(dtype)
    v = (torch.randn(n_pages, n_kv, page, d, device="cuda") * 0.5).to(dtype)
    # pages of one sequence are scattered over the pool, as they are after slots were reused
    perm = torch.randperm(n_pages, device="cuda").to(torch.int32).view(B, per_seq).contiguous()
    return k, v, perm


def _decode_splits(B, n_kv, max_len, page, d, fused):
    """How the attention part cuts the keys of a decoding step (libllm_b200/parts/builtin.cc)."""
    import torch
    from ..csrc import ops
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    pairs = max(1, B * n_kv)
    if fused:
        slots = sms * ops.attention_decode_tc_ctas_per_sm(d)
        return 0, max(1, min(slots // pairs, max(1, max_len // page)))
    want = max(1, (8 * sms + pairs - 1) // pairs)
    n_splits = max(1, min(want, max(1, max_len // (2 * page))))
    chunk = (max_len + n_splits - 1) // n_splits
    chunk = (chunk + page - 1) // page * page
    return chunk, max(1, (max_len + chunk - 1) // chunk)


def bench_attention_decode(args, timer):
    import torch
    from ..csrc import ops
    B, ctx, nH, nKV, d = args.batch, args.context, args.heads, args.kv_heads, args.head_dim
    k, v, table = _paged_cache(B, ctx, nKV, d)
    pos = torch.full((B,), ctx - 1, dtype=torch.int32, device="cuda")
    scale = 1.0 / math.sqrt(d)
    nbytes = 2 * B * ctx * nKV * d * 2 + 2 * B * nH * d * 2
    if args.separate:
        q = torch.randn(B, nH * d, device="cuda").to(torch.bfloat16)
        out = torch.empty_like(q)
        chunk, n_splits = _decode_splits(B, nKV, table.shape[1] * 64, 64, d, fused=False)
        ws_o = torch.empty(B * nH * n_splits * d, dtype=torch.float32, device="cuda")
        ws_ml = torch.empty(B * nH * n_splits * 2, dtype=torch.float32, device="cuda")

        def fn():
            ops.attention_decode(q, out, k, v, pos, table, nH, nKV, d, 64, chunk, n_splits, None, scale,
                                 ws_o if n_splits > 1 else None, ws_ml if n_splits > 1 else None)
        name = "attention_decode (FMA kernel + join kernel)"
    else:
        qkv = torch.randn(B, (nH + 2 * nKV) * d, device="cuda")
        out = torch.empty(B, nH * d, device="cuda", dtype=torch.bfloat16)
        ang = torch.arange(ctx + 1, device="cuda", dtype=torch.float64)[:, None] * \
            (10000.0 ** (-torch.arange(0, d, 2, device="cuda", dtype=torch.float64) / d))[None]
        rope = torch.cat([ang.cos(), ang.sin()], 1).float().contiguous()
        chunk, n_splits = _decode_splits(B, nKV, table.shape[1] * 64, 64, d, fused=True)
        ws_o = torch.empty(B * nH * n_splits * d, dtype=torch.float32, device="cuda")
        ws_ml = torch.empty(B * nH * n_splits * 2, dtype=torch.float32, device="cuda")
        counters = torch.zeros(B * nKV, dtype=torch.int32, device="cuda")

        def fn():
            ops.attention_decode_tc(qkv, out, rope, k, v, pos, table, nH, nKV, d, 64, chunk, n_splits, None, scale,
                                    True, ws_o, ws_ml, counters, max_len=table.shape[1] * 64)
        name = "attention_decode_tc (rotation, append, attention, join)"
    us = timer.run(fn)
    report(name, us, bytes_moved=nbytes, flops=4 * B * nH * ctx * d, batch=B, context=ctx, heads=nH, kv_heads=nKV,
           head_dim=d, chunk=chunk, splits=n_splits)


def bench_attention_prefill(args, timer):
    import torch
    from ..csrc import ops
    T, nH, nKV, d = args.tokens, args.heads, args.kv_heads, args.head_dim
    B = args.batch
    k, v, table = _paged_cache(B, T, nKV, d)
    q = torch.randn(B * T, nH * d, device="cuda").to(torch.bfloat16)
    out = torch.empty_like(q)
    tok_seq = torch.arange(B, device="cuda", dtype=torch.int32).repeat_interleave(T).contiguous()
    tok_pos = torch.arange(T, device="cuda", dtype=torch.int32).repeat(B).contiguous()
    seq_start = (torch.arange(B + 1, device="cuda", dtype=torch.int32) * T).contiguous()
    seq_past = torch.zeros(B, device="cuda", dtype=torch.int32)
    scale = 1.0 / math.sqrt(d)
    use_fast = not args.generic and ops.attention_prefill_supported(d, 64)
    use_tc = use_fast and not args.mma_sync and ops.attention_prefill_tc_supported(d, 64)

    def fn():
        if use_tc:
            ops.attention_prefill_tc(q, out, k, v, seq_start, seq_past, table, B, T, nH, nKV, d, 64, None, scale, args.form)
        elif use_fast:
            ops.attention_prefill(q, out, k, v, seq_start, seq_past, table, B, T, nH, nKV, d, 64, None, scale)
        else:
            ops.attention_generic(q, out, k, v, tok_seq, tok_pos, table, nH, nKV, d, 64, None, scale)
    us = timer.run(fn)
    report("attention_prefill_tc" if use_tc else ("attention_prefill" if use_fast else "attention_generic"), us,
           flops=4 * B * nH * d * T * (T + 1) // 2, batch=B, tokens=T, heads=nH, kv_heads=nKV, head_dim=d,
           **({"form": args.form} if use_tc else {}))


def bench_chain_layer(args, timer):
    """A layer's products and norms between two attentions (output projection, add + norm, gate|up +
    SwiGLU, down, add + norm, q|k|v) as ONE chained launch against the same six as launches of their
    own, and the times the chained kernel records inside itself (the device's nanosecond clock)."""
    import ctypes
    import torch
    from ..csrc import build, ops
    T, H, I = args.m, args.hidden, args.intermediate
    Kq = args.heads * args.head_dim
    Nq = (args.heads + 2 * args.kv_heads) * args.head_dim
    bf = torch.bfloat16

    def rnd(shape, std=1.0, dt=bf):
        return (torch.randn(shape, device="cuda") * std).to(dt)
    attn, wo, wgu = rnd((T, Kq)), rnd((H, Kq), Kq ** -0.5), rnd((2 * I, H), H ** -0.5)
    wd, wqkv = rnd((H, I), I ** -0.5), rnd((Nq, H), H ** -0.5)
    n1, n2 = torch.ones(H, device="cuda"), torch.ones(H, device="cuda")
    resid = rnd((T, H), dt=torch.float32)
    po, pd, pq = (ops.gemm_tc_suggest_parts(T, H, Kq), ops.gemm_tc_suggest_parts(T, H, I), ops.gemm_tc_suggest_parts(T, Nq, H))
    o_parts = torch.empty((po, T, H), dtype=torch.float32, device="cuda")
    d_parts = torch.empty((pd, T, H), dtype=torch.float32, device="cuda")
    qkv = torch.empty((pq, T, Nq), dtype=torch.float32, device="cuda")
    h1, h2 = torch.empty((T, H), dtype=bf, device="cuda"), torch.empty((T, H), dtype=bf, device="cuda")
    m = torch.empty((T, I), dtype=bf, device="cuda")
    counters = torch.zeros(16, dtype=torch.int32, device="cuda")
    jobs = [ops.chain_product(attn, wo, o_parts), ops.chain_norm(resid, o_parts, n1, 1e-5, h1, deps=(0, -1)),
            ops.chain_product(h1, wgu, m, swiglu=True, deps=(1, -1)), ops.chain_product(m, wd, d_parts, deps=(2, -1)),
            ops.chain_norm(resid, d_parts, n2, 1e-5, h2, deps=(3, 1)), ops.chain_product(h2, wqkv, qkv, deps=(4, -1))]

    def separate():
        ops.gemm_tc(attn, wo, o_parts)
        ops.add_rmsnorm(resid, o_parts, n1, 1e-5, h1)
        ops.gemm_tc(h1, wgu, m, swiglu=True)
        ops.gemm_tc(m, wd, d_parts)
        ops.add_rmsnorm(resid, d_parts, n2, 1e-5, h2)
        ops.gemm_tc(h2, wqkv, qkv)
    nbytes = 2 * (wo.numel() + wgu.numel() + wd.numel() + wqkv.numel())
    report("six launches", timer.run(separate), bytes_moved=nbytes, m=T)
    report("one chained launch", timer.run(lambda: ops.gemm_chain(jobs, counters)), bytes_moved=nbytes, m=T)
    # the kernel's own account of one launch
    names = ["o", "add+norm", "gate|up+swiglu", "down", "add+norm", "q|k|v"]
    tiles = [((H + 127) // 128) * po, T, (I + 63) // 64, ((H + 127) // 128) * pd, T, ((Nq + 127) // 128) * pq]
    total = sum(tiles)
    grid = min(total, torch.cuda.get_device_properties(0).multi_processor_count)
    trace = torch.zeros(total + 10 * grid + 256, dtype=torch.int64, device="cuda")
    lib = build.load("gemm_chain")
    lib.llm_gemm_chain_trace.argtypes = [ctypes.c_void_p]
    if timer.flusher is not None:
        timer.flusher.fill_(1)
    torch.cuda.synchronize()
    lib.llm_gemm_chain_trace(ctypes.c_void_p(trace.data_ptr()))
    try:
        ops.gemm_chain(jobs, counters)
        torch.cuda.synchronize()
    finally:
        lib.llm_gemm_chain_trace(ctypes.c_void_p(0))
    t = trace.cpu().numpy()
    per = t[total:total + 10 * grid].reshape(grid, 10)
    start = int(per[:, 8].min())
    base, phases = 0, []
    for j, n in enumerate(tiles):
        done = t[base:base + n]
        base += n
        seen = per[:, j][per[:, j] > 0]
        phases.append(dict(job=names[j], tiles=n,
                           inputs_seen_us=[round((int(seen.min()) - start) / 1e3, 2), round((int(seen.max()) - start) / 1e3, 2)] if len(seen) else None,
                           tiles_done_us=[round((int(done.min()) - start) / 1e3, 2), round((int(done.max()) - start) / 1e3, 2)]))
    print(json.dumps({"chained launch, times after its first CTA started": phases}), flush=True)


def bench_add_rmsnorm(args, timer):
    import torch
    from ..csrc import ops
    T, H, P = args.m, args.hidden, max(1, args.parts)
    resid = torch.randn(T, H, device="cuda")
    delta = torch.randn(T, H, device="cuda") if P == 1 else torch.randn(P, T, H, device="cuda")
    w = torch.ones(H, device="cuda")
    out = torch.empty(T, H, device="cuda", dtype=torch.bfloat16)
    us = timer.run(lambda: ops.add_rmsnorm(resid, delta, w, 1e-5, out))
    report("add_rmsnorm", us, bytes_moved=T * H * (4 + 4 * P + 4 + 2), m=T, hidden=H, parts=P)


def bench_sampling(args, timer):
    import torch
    from ..csrc import ops
    B, V = args.batch, args.vocab
    logits = torch.randn(B, V, device="cuda")
    out = torch.empty(B, dtype=torch.int32, device="cuda")
    uni = torch.rand(B, device="cuda")
    us = timer.run(lambda: ops.argmax(logits, out))
    report("argmax", us, bytes_moved=B * V * 4, batch=B, vocab=V)
    us = timer.run(lambda: ops.sample(logits, 0.8, 50, 0.8, uni, out))
    report("sample_top_k50_top_p0.8", us, bytes_moved=B * V * 4, batch=B, vocab=V)


def bench_gemm(args, timer):
    """The library product (cuBLAS, here through torch) that prompts use, for comparison."""
    import torch
    M, N, K = args.m, args.n, args.k
    x = torch.randn(M, K, device="cuda").to(torch.bfloat16)
    w = (torch.randn(N, K, device="cuda") * 0.02).to(torch.bfloat16)
    us = timer.run(lambda: torch.mm(x, w.t()))
    report("library_gemm", us, flops=2 * M * N * K, bytes_moved=2 * (M * K + N * K + M * N), m=M, n=N, k=K)


KERNELS = {"gemv": bench_gemv, "layer_products": bench_layer_products, "attention_decode": bench_attention_decode,
           "attention_prefill": bench_attention_prefill, "add_rmsnorm": bench_add_rmsnorm,
           "sampling": bench_sampling, "gemm": bench_gemm, "chain_layer": bench_chain_layer}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="kernel_bench", description=__doc__.split("\n\n")[0])
    ap.add_argument("kernel", choices=sorted(KERNELS))
    ap.add_argument("--m", type=int, default=8, help="tokens in the step")
    ap.add_argument("--n", type=int, default=128256)
    ap.add_argument("--k", type=int, default=2048)
    ap.add_argument("--swiglu", action="store_true")
    ap.add_argument("--parts", type=int, default=1, help="add_rmsnorm: partial products the norm adds up first")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=2048)
    ap.add_argument("--tokens", type=int, default=2048)
    ap.add_argument("--hidden", type=int, default=2048)
    ap.add_argument("--intermediate", type=int, default=8192)
    ap.add_argument("--vocab", type=int, default=128256)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--head-dim", type=int, default=64)
    ap.add_argument("--tc", action="store_true", help="gemv, layer_products: time the tcgen05 product")
    ap.add_argument("--library", action="store_true", help="gemv, layer_products: time the library product instead")
    ap.add_argument("--separate", action="store_true",
                    help="attention_decode: time the FMA kernel with its join kernel instead of the fused one")
    ap.add_argument("--mma-sync", action="store_true", help="attention_prefill: time the mma.sync kernel")
    ap.add_argument("--form", type=int, default=0, choices=[0, 1, 2],
                    help="attention_prefill on tcgen05: 1 CTAs of 128 rows, 2 of 256 rows, 0 the library's choice")
    ap.add_argument("--generic", action="store_true", help="attention_prefill: time the general kernel")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--no-flush", action="store_true", help="do not write a buffer larger than L2 between launches")
    args = ap.parse_args(argv)
    import torch
    if not torch.cuda.is_available():
        print("kernel_bench needs a CUDA device", file=sys.stderr)
        return 1
    timer = Timer(max(1, args.iters), max(0, args.warmup), flush=not args.no_flush)
    KERNELS[args.kernel](args, timer)
    return 0


if __name__ == "__main__":
    sys.exit(main())
