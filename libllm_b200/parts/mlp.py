"""Dense SwiGLU feed-forward."""
from __future__ import annotations

from typing import List

import torch

from ..csrc import ops
from ..weights.state_map import TensorNeed
from . import fast
from .base import FeedForward, StepContext
from .linear import linear
from .registry import part


@part("feed_forward", "swiglu")
class SwiGLU(FeedForward):
    """down(silu(gate(x)) * up(x)), no biases (src/libllm/llama.cc:81-98).  Gate and up
    are one stacked product, gate rows first (tools/llama_exporter.py:73-77); the
    activation a/(1+exp(-a)) times up is computed in 32-bit (src/flint/cuda/swiglu.cu:44-49)."""

    def tensor_needs(self) -> List[TensorNeed]:
        s = self.spec
        return [TensorNeed(s.gate, (s.intermediate, s.hidden)), TensorNeed(s.up, (s.intermediate, s.hidden)),
                TensorNeed(s.down, (s.hidden, s.intermediate))]

    def load(self, fetch) -> None:
        needs = self.tensor_needs()
        self.w_gate_up = torch.cat([fetch(needs[0]), fetch(needs[1])], dim=0).contiguous()
        self.w_down = fetch(needs[2])

    def kernel_families(self) -> List[str]:
        return ["elementwise"] + fast.product_families(self.env.dtype)

    def forward(self, ctx: StepContext, x: torch.Tensor) -> torch.Tensor:
        m = None
        if x.dtype == torch.bfloat16:
            m = fast.small_batch_linear(x, self.w_gate_up, ctx.dtype, swiglu=True)
            if m is None:
                m = fast.fused_gate_up(x, self.w_gate_up, ctx.dtype)
        if m is not None:
            return linear(m, self.w_down, out_dtype=torch.float32, parts_ok=True)
        gu = linear(x, self.w_gate_up, out_dtype=torch.float32)
        m = torch.empty((x.shape[0], self.spec.intermediate), dtype=ctx.dtype, device=ctx.device)
        ops.swiglu(gu, m)
        return linear(m, self.w_down, out_dtype=torch.float32, parts_ok=True)
