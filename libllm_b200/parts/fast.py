"""Switchboard of the fast bfloat16 kernels: each entry returns None when the kernel
does not take the case, and the caller then uses the general kernel.  A kernel can be
switched off by an environment variable to compare it with the general one."""
from __future__ import annotations

import os
from typing import List, Optional, Tuple

import torch

from ..csrc import ops
from ..errors import UnsupportedError

ENABLED = {
    "gemv": os.environ.get("LIBLLM_B200_NO_GEMV") is None,
    "decode_attention": os.environ.get("LIBLLM_B200_NO_DECODE_ATTENTION") is None,
    "prefill_attention": os.environ.get("LIBLLM_B200_NO_PREFILL_ATTENTION") is None,
    "gemm_tc": os.environ.get("LIBLLM_B200_NO_GEMM_TC") is None,
    "prefill_attention_tc": os.environ.get("LIBLLM_B200_NO_PREFILL_ATTENTION_TC") is None,
    "decode_attention_tc": os.environ.get("LIBLLM_B200_NO_DECODE_ATTENTION_TC") is None,
}
PRODUCT = os.environ.get("LIBLLM_B200_PRODUCT", "tc")           # "gemv": never the tcgen05 kernel
TC_TOKENS = int(os.environ.get("LIBLLM_B200_TC_TOKENS", "256"))
FUSED_GATE_UP_TOKENS = int(os.environ.get("LIBLLM_B200_FUSED_GATE_UP_TOKENS", "1024"))
FUSED_GATE_UP_MAX_K = 3072
SM_COUNT = 148
# Steps of up to this many tokens take the mma.sync weight streamer (csrc/gemv.cu) instead of the
# tcgen05 product.  Off by default: inside a step the two are equally fast at 8 tokens, but the
# streamer reads its tokens through L1 and slows down when a kernel with much shared memory runs
# beside it, and above 16 tokens it falls behind (661 us against 181 us for a layer's products at 64).
GEMV_TOKENS = int(os.environ.get("LIBLLM_B200_GEMV_TOKENS", "0"))


def product_families(dtype: torch.dtype) -> List[str]:
    """Kernel families that the products of an engine of this type launch (compiled when the model
    is built; a family that a rare case needs beyond these is compiled when that case comes)."""
    fams = ["gemm_plain"]                      # the 32-bit path; with bfloat16, products with a bias
    if dtype == torch.bfloat16:
        if ENABLED["gemm_tc"] and PRODUCT == "tc":
            fams.append("gemm_tc")
        if ENABLED["gemv"] and (GEMV_TOKENS > 0 or PRODUCT != "tc"):
            fams.append("gemv")
    return fams


def attention_families(spec, dtype: torch.dtype, page_size: int) -> List[str]:
    """The same for an attention part with this head size, grouping and page size."""
    fams = ["rope", "attention_generic"]
    if dtype != torch.bfloat16:
        return fams
    d, group = spec.head_dim, spec.n_heads // spec.n_kv_heads
    tiled = page_size == 64 and d % 16 == 0 and 16 <= d <= 128
    if ENABLED["prefill_attention_tc"] and page_size == 64 and d in (64, 128):
        fams.append("attention_prefill_tc")
    elif ENABLED["prefill_attention"] and tiled:
        fams.append("attention_prefill")
    fused = ENABLED["decode_attention_tc"] and tiled and group <= 16 and not spec.bias and spec.position is not None
    if fused:
        fams.append("attention_decode_tc")
    elif ENABLED["decode_attention"] and d in (16, 32, 64, 128) and group in (1, 2, 3, 4, 8):
        fams.append("attention_decode")
    return fams


def small_batch_linear(x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype, swiglu: bool = False,
                       parts_ok: bool = False) -> Optional[torch.Tensor]:
    """The product for steps of few tokens, where reading the weights once is what costs: the
    mma.sync weight streamer up to ``GEMV_TOKENS`` tokens, the tcgen05 kernel up to ``TC_TOKENS``.  With ``parts_ok`` the result may come
    as [parts, T, N] partial products over K (32-bit) that the caller adds: matrices with few
    rows are cut along K so that every SM has work."""
    T = x.shape[0]
    n = w.shape[0] // 2 if swiglu else w.shape[0]
    use_gemv = ENABLED["gemv"] and T <= GEMV_TOKENS and ops.gemv_supported(x, w)
    if PRODUCT == "tc" and ENABLED["gemm_tc"] and T <= TC_TOKENS and not use_gemv and ops.gemm_tc_supported(x, w):
        if parts_ok and not swiglu and out_dtype == torch.float32:
            parts = ops.gemm_tc_suggest_parts(T, n, x.shape[1])
            if parts > 1:
                return ops.gemm_tc(x, w, torch.empty((parts, T, n), dtype=out_dtype, device=x.device))
        return ops.gemm_tc(x, w, torch.empty((T, n), dtype=out_dtype, device=x.device), swiglu)
    if not use_gemv:
        return None
    if parts_ok and not swiglu and out_dtype == torch.float32:
        parts = ops.gemv_suggest_parts(T, n, x.shape[1])
        if parts > 1:
            out = torch.empty((parts, T, n), dtype=out_dtype, device=x.device)
            return ops.gemv_bf16(x, w, out)
    out = torch.empty((T, n), dtype=out_dtype, device=x.device)
    return ops.gemv_bf16(x, w, out, swiglu)


def fused_gate_up(x: torch.Tensor, w_gate_up: torch.Tensor, out_dtype: torch.dtype) -> Optional[torch.Tensor]:
    """silu(gate) * up of a prompt step in one launch of the tcgen05 product (two accumulators per
    tile), where that beats the library product followed by a SwiGLU pass: measured at 2,048 tokens,
    129 us against 146 us at K = 2,048, but 403 us against 379 us at K = 4,096 (the separate pass
    costs the same whatever K is, the product's shortfall grows with K)."""
    T, K = x.shape
    if not (ENABLED["gemm_tc"] and PRODUCT == "tc" and T >= FUSED_GATE_UP_TOKENS and K <= FUSED_GATE_UP_MAX_K
            and ops.gemm_tc_supported(x, w_gate_up)):
        return None
    return ops.gemm_tc(x, w_gate_up, torch.empty((T, w_gate_up.shape[0] // 2), dtype=out_dtype, device=x.device), True)


def decode_split(n_seqs: int, n_kv: int, max_kv_len: int, page_size: int) -> Tuple[int, int]:
    """(chunk, n_splits) for decode attention: enough CTAs to fill the GPU about eight
    times over at the longest length, runs of at least two pages, the same for every step of a captured graph
    (it depends on the graph's bound on the length, not on the lengths themselves)."""
    pairs = max(1, n_seqs * n_kv)
    want = max(1, (8 * SM_COUNT + pairs - 1) // pairs)
    most = max(1, max_kv_len // (2 * page_size))
    n_splits = max(1, min(want, most))
    chunk = (max_kv_len + n_splits - 1) // n_splits
    chunk = (chunk + page_size - 1) // page_size * page_size
    n_splits = (max_kv_len + chunk - 1) // chunk
    return chunk, max(1, n_splits)


_counters = {}


COUNTERS = 1 << 18


def _zero_counters(device, n: int) -> torch.Tensor:
    """int32 zeros in which the fused decode attention counts finished splits (it leaves them zero).
    One buffer per device for good: captured steps keep its address."""
    if n > COUNTERS:
        raise UnsupportedError(f"fused decode attention: {n} (sequence, kv head) pairs in one step, "
                               f"{COUNTERS} are provided for")
    t = _counters.get(device)
    if t is None:
        t = _counters[device] = torch.zeros(COUNTERS, dtype=torch.int32, device=device)
    return t


def fused_decode_possible(ctx, cache, spec) -> bool:
    group = spec.n_heads // spec.n_kv_heads
    return bool(ctx.decode_only and ENABLED["decode_attention_tc"] and ctx.dtype == torch.bfloat16 and cache is not None
                and ops.attention_decode_tc_supported(spec.head_dim, cache.page_size, group))


def fused_decode_splits(n_seqs: int, n_kv: int, max_kv_len: int, page_size: int, head_dim: int = 64) -> int:
    """Key splits per sequence for the fused decode attention: as many as fill the GPU once (all
    CTAs resident together: no second, partly filled wave), each of at least a page at the longest
    length.  The kernel cuts every sequence's own length into that many runs, so the number
    depends on the batch and on the graph's bound on the length, not on the lengths themselves."""
    pairs = max(1, n_seqs * n_kv)
    slots = SM_COUNT * ops.attention_decode_tc_ctas_per_sm(head_dim)
    return max(1, min(slots // pairs, max(1, max_kv_len // page_size)))


def fused_decode_attention(ctx, qkv: torch.Tensor, cache, spec, table: torch.Tensor,
                           scale: float) -> Optional[torch.Tensor]:
    """Rotation, cache append and attention of a decode-only step in one launch; None when the
    kernel does not take the case (then the parts run one after another).  ``qkv`` is the 32-bit
    stacked product, [T, W] or [parts, T, W]."""
    if not fused_decode_possible(ctx, cache, spec) or qkv.dtype != torch.float32:
        return None
    max_len = max(ctx.max_kv_len, 1)
    n_splits = fused_decode_splits(ctx.n_seqs, spec.n_kv_heads, max_len, cache.page_size, spec.head_dim)
    dev = qkv.device
    out = torch.empty((ctx.n_tokens, spec.n_heads * spec.head_dim), dtype=torch.bfloat16, device=dev)
    ws_o = ws_ml = counters = None
    if n_splits > 1:
        ws_o = torch.empty(ctx.n_seqs * spec.n_heads * n_splits * spec.head_dim, dtype=torch.float32, device=dev)
        ws_ml = torch.empty(ctx.n_seqs * spec.n_heads * n_splits * 2, dtype=torch.float32, device=dev)
        counters = _zero_counters(dev, ctx.n_seqs * spec.n_kv_heads)
    return ops.attention_decode_tc(qkv, out, table, cache.k, cache.v, ctx.tok_pos, cache.page_table, spec.n_heads,
                                   spec.n_kv_heads, spec.head_dim, cache.page_size, 0, n_splits, spec.window,
                                   scale, cache.writes, ws_o, ws_ml, counters, max_len=max_len)


def attention(ctx, q: torch.Tensor, cache, spec, scale: float) -> Optional[torch.Tensor]:
    if q.dtype != torch.bfloat16:
        return None
    group = spec.n_heads // spec.n_kv_heads
    if ctx.decode_only and ENABLED["decode_attention"] and ops.attention_decode_supported(spec.head_dim, group):
        chunk, n_splits = decode_split(ctx.n_seqs, spec.n_kv_heads, max(ctx.max_kv_len, 1), cache.page_size)
        out = torch.empty((ctx.n_tokens, spec.n_heads * spec.head_dim), dtype=q.dtype, device=q.device)
        ws_o = ws_ml = None
        if n_splits > 1:
            ws_o = torch.empty(ctx.n_seqs * spec.n_heads * n_splits * spec.head_dim, dtype=torch.float32, device=q.device)
            ws_ml = torch.empty(ctx.n_seqs * spec.n_heads * n_splits * 2, dtype=torch.float32, device=q.device)
        # In a decode-only step token i is sequence i, so tok_pos is the per-sequence position.
        return ops.attention_decode(q, out, cache.k, cache.v, ctx.tok_pos, cache.page_table, spec.n_heads,
                                    spec.n_kv_heads, spec.head_dim, cache.page_size, chunk, n_splits, spec.window,
                                    scale, ws_o, ws_ml)
    # (the head sizes are asked here first: asking the library would compile it for a model that never uses it)
    if ENABLED["prefill_attention_tc"] and spec.head_dim in (64, 128) and \
            ops.attention_prefill_tc_supported(spec.head_dim, cache.page_size):
        out = torch.empty((ctx.n_tokens, spec.n_heads * spec.head_dim), dtype=q.dtype, device=q.device)
        return ops.attention_prefill_tc(q, out, cache.k, cache.v, ctx.seq_start, ctx.seq_past, cache.page_table,
                                        ctx.n_seqs, ctx.max_q_len, spec.n_heads, spec.n_kv_heads, spec.head_dim,
                                        cache.page_size, spec.window, scale)
    if ENABLED["prefill_attention"] and ops.attention_prefill_supported(spec.head_dim, cache.page_size):
        out = torch.empty((ctx.n_tokens, spec.n_heads * spec.head_dim), dtype=q.dtype, device=q.device)
        return ops.attention_prefill(q, out, cache.k, cache.v, ctx.seq_start, ctx.seq_past, cache.page_table,
                                     ctx.n_seqs, ctx.max_q_len, spec.n_heads, spec.n_kv_heads, spec.head_dim,
                                     cache.page_size, spec.window, scale)
    return None
