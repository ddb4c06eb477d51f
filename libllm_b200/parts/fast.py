"""Switchboard of the fast bfloat16 kernels: each entry returns None when the kernel
does not take the case, and the caller then uses the general kernel.  A kernel can be
switched off by an environment variable to compare it with the general one."""
from __future__ import annotations

import os
from typing import Optional, Tuple

import torch

from ..csrc import ops

ENABLED = {
    "gemv": os.environ.get("LIBLLM_B200_NO_GEMV") is None,
    "decode_attention": os.environ.get("LIBLLM_B200_NO_DECODE_ATTENTION") is None,
    "prefill_attention": os.environ.get("LIBLLM_B200_NO_PREFILL_ATTENTION") is None,
}
SM_COUNT = 148
# Above this many tokens the library product is faster than the weight streamer (measured at the
# layer sizes of Llama-3.2-1B: 181 us against 661 us for a layer's products at 64 tokens).
GEMV_TOKENS = int(os.environ.get("LIBLLM_B200_GEMV_TOKENS", "16"))


def small_batch_linear(x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype, swiglu: bool = False,
                       parts_ok: bool = False, prefetch: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
    """The weight-streaming product for steps of up to 64 tokens.  With ``parts_ok`` the
    result may come as [parts, T, N] partial products over K (32-bit) that the caller adds:
    matrices with few rows are cut along K so that every SM has work."""
    if not ENABLED["gemv"] or x.shape[0] > GEMV_TOKENS or not ops.gemv_supported(x, w):
        return None
    n = w.shape[0] // 2 if swiglu else w.shape[0]
    if parts_ok and not swiglu and out_dtype == torch.float32:
        parts = ops.gemv_suggest_parts(x.shape[0], n, x.shape[1])
        if parts > 1:
            out = torch.empty((parts, x.shape[0], n), dtype=out_dtype, device=x.device)
            return ops.gemv_bf16(x, w, out, prefetch=prefetch)
    out = torch.empty((x.shape[0], n), dtype=out_dtype, device=x.device)
    return ops.gemv_bf16(x, w, out, swiglu, prefetch=prefetch)


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
    if ENABLED["prefill_attention"] and ops.attention_prefill_supported(spec.head_dim, cache.page_size):
        out = torch.empty((ctx.n_tokens, spec.n_heads * spec.head_dim), dtype=q.dtype, device=q.device)
        return ops.attention_prefill(q, out, cache.k, cache.v, ctx.seq_start, ctx.seq_past, cache.page_table,
                                     ctx.n_seqs, ctx.max_q_len, spec.n_heads, spec.n_kv_heads, spec.head_dim,
                                     cache.page_size, spec.window, scale)
    return None
