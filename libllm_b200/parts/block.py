"""How a mixer and a feed-forward join the residual stream."""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .base import Block, LayerCache, Mixer, Part, ResidualStream, StepContext
from .registry import build_part, part


@part("block", "prenorm")
class PreNormBlock(Block):
    """h = x + mixer(norm1(x)); out = h + ff(norm2(h)) (src/libllm/llama.cc:251-267).
    Each addition is left pending on the stream and applied, in 32-bit, by the next norm."""

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.mixer_norm = build_part("norm", spec.mixer_norm, env)
        self.mixer = build_part("mixer", spec.mixer, env)
        self.ff_norm = build_part("norm", spec.ff_norm, env)
        self.ff = build_part("feed_forward", spec.ff, env)

    def parts(self) -> List[Part]:
        return [self.mixer_norm, self.mixer, self.ff_norm, self.ff]

    def mixer_part(self) -> Optional[Mixer]:
        return self.mixer

    def tensor_needs(self):
        return [n for p in self.parts() for n in p.tensor_needs()]

    def load(self, fetch) -> None:
        for p in self.parts():
            p.load(fetch)

    def kernel_families(self) -> List[str]:
        return sorted({f for p in self.parts() for f in p.kernel_families()})

    def forward(self, ctx: StepContext, stream: ResidualStream, cache: Optional[LayerCache],
                state: Optional[Dict[str, torch.Tensor]]) -> None:
        h = self.mixer_norm.forward(ctx, stream)
        stream.pending = self.mixer.forward(ctx, h, cache, state)
        h = self.ff_norm.forward(ctx, stream)
        stream.pending = self.ff.forward(ctx, h)
