"""Grouped-query attention over the paged cache."""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

from ..csrc import ops
from ..errors import ConfigError, UnsupportedError
from ..weights.state_map import TensorNeed
from . import fast
from .base import CacheNeed, LayerCache, Mixer, StepContext
from .linear import linear
from .registry import build_part, part


@part("mixer", "attention")
class Attention(Mixer):
    """q, k, v from one stacked product, rotation of q and k, append to the cache,
    softmax(q k^T / sqrt(d)) v per head with a causal mask, output projection
    (src/libllm/llama.cc:178-225).  The stacked matrix is [Wq; Wk; Wv] as the
    reference's exporter builds it (tools/llama_exporter.py:64-71), made here when the
    weights are loaded."""

    def __init__(self, spec, env):
        super().__init__(spec, env)
        s = spec
        if s.n_heads % s.n_kv_heads:
            raise ConfigError(f"attention: {s.n_heads} heads are not a multiple of {s.n_kv_heads} groups")
        if s.head_dim % 16 or not 16 <= s.head_dim <= 256:
            raise UnsupportedError(f"attention: head size {s.head_dim} is not supported "
                                   "(multiples of 16 from 16 to 256)")
        self.position = build_part("position", s.position, env) if s.position is not None else None
        self.scale = s.scale if s.scale is not None else 1.0 / math.sqrt(s.head_dim)
        self.q_width = s.n_heads * s.head_dim
        self.kv_width = s.n_kv_heads * s.head_dim

    def tensor_needs(self) -> List[TensorNeed]:
        s = self.spec
        needs = [TensorNeed(s.q, (self.q_width, s.hidden)), TensorNeed(s.k, (self.kv_width, s.hidden)),
                 TensorNeed(s.v, (self.kv_width, s.hidden)), TensorNeed(s.o, (s.hidden, self.q_width))]
        if s.bias:
            for n, w in ((s.q, self.q_width), (s.k, self.kv_width), (s.v, self.kv_width)):
                needs.append(TensorNeed(n[:-len("weight")] + "bias", (w,), role="vector"))
        return needs

    def load(self, fetch) -> None:
        needs = self.tensor_needs()
        self.w_qkv = torch.cat([fetch(n) for n in needs[:3]], dim=0).contiguous()
        self.w_o = fetch(needs[3])
        if self.position is not None:
            self.position.load(fetch)
        self.b_qkv = None
        if self.spec.bias:
            self.b_qkv = torch.cat([fetch(n).to(torch.float32) for n in needs[4:7]]).contiguous()

    def kernel_families(self) -> List[str]:
        return fast.product_families(self.env.dtype) + fast.attention_families(self.spec, self.env.dtype, self.env.page_size)

    def cache_need(self) -> Optional[CacheNeed]:
        s = self.spec
        return CacheNeed("window" if s.window else "full", s.n_kv_heads, s.head_dim, s.window)

    def forward(self, ctx: StepContext, x: torch.Tensor, cache: Optional[LayerCache],
                state: Optional[Dict[str, torch.Tensor]]) -> torch.Tensor:
        s = self.spec
        # The products hand over 32-bit results: q and k are rounded to the engine's
        # type once, after the rotation, and the residual addition gets an unrounded term.
        table = getattr(self.position, "table", None) if self.position is not None else None
        fused = table is not None and self.b_qkv is None and fast.fused_decode_possible(ctx, cache, s)
        qkv = linear(x, self.w_qkv, self.b_qkv, out_dtype=torch.float32, parts_ok=fused)
        if self.position is None:
            raise UnsupportedError("attention without a position encoding is not built")
        if fused:
            out = fast.fused_decode_attention(ctx, qkv, cache, s, table, self.scale)
            if out is not None:
                return linear(out, self.w_o, out_dtype=torch.float32, parts_ok=True)
            raise UnsupportedError("attention: the fused decode kernel refused a step it had accepted")
        q = torch.empty((ctx.n_tokens, self.q_width), dtype=ctx.dtype, device=ctx.device)
        ops.rope_cache_write(qkv, q, s.n_heads, s.n_kv_heads, s.head_dim, self.position.table,
                             ctx.tok_seq, ctx.tok_pos, cache.page_table, cache.k, cache.v,
                             cache.page_size, cache.writes)
        out = fast.attention(ctx, q, cache, s, self.scale)
        if out is None:
            out = torch.empty((ctx.n_tokens, self.q_width), dtype=ctx.dtype, device=ctx.device)
            ops.attention_generic(q, out, cache.k, cache.v, ctx.tok_seq, ctx.tok_pos, cache.page_table,
                                  s.n_heads, s.n_kv_heads, s.head_dim, cache.page_size, s.window, self.scale)
        return linear(out, self.w_o, out_dtype=torch.float32, parts_ok=True)
