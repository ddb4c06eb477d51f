"""RMSNorm with the pending residual addition folded in."""
from __future__ import annotations

from typing import List, Optional

import torch

from ..csrc import ops
from ..weights.state_map import TensorNeed
from .base import Norm, ResidualStream, StepContext
from .registry import part


@part("norm", "rmsnorm")
class RMSNorm(Norm):
    """y = x * w / sqrt(mean(x^2) + eps), sums and scaling in 32-bit
    (src/flint/cpu/normalizations.cc:52-64, src/flint/cuda/rms_norm.cu:59-75).  Before
    the norm the stream's pending addition is applied in 32-bit: the reference's
    separate residual add (src/libllm/llama.cc:252-266)."""

    def tensor_needs(self) -> List[TensorNeed]:
        return [TensorNeed(self.spec.weight, (self.spec.size,), role="vector")]

    def load(self, fetch) -> None:
        self.weight = fetch(self.tensor_needs()[0]).to(torch.float32).contiguous()

    def kernel_families(self) -> List[str]:
        return ["elementwise"]

    def forward(self, ctx: StepContext, stream: ResidualStream,
                rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        n = stream.resid.shape[0] if rows is None else rows.numel()
        out = torch.empty((n, self.spec.size), dtype=ctx.dtype, device=ctx.device)
        ops.add_rmsnorm(stream.resid, stream.pending, self.weight, self.spec.eps, out, rows)
        if rows is None:
            stream.pending = None
        return out
