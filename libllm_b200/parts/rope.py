"""Rotary position encoding: frequencies (with the "llama3" rescaling) and the table."""
from __future__ import annotations

import math
from typing import List

import torch

from ..errors import ConfigError
from .base import PositionEncoding
from .registry import part


def rotary_frequencies(rotary_dim: int, theta: float, scaling) -> List[float]:
    """f_i = theta^(-2i/d) for i < d/2.  With llama3 scaling a frequency whose wavelength
    2*pi/f is shorter than original/high_freq_factor is kept, one longer than
    original/low_freq_factor is divided by ``factor``, and between them the two are
    blended linearly in original/wavelength.  The reference takes the finished cos/sin
    table from the checkpoint's own rotary module (tools/llama_exporter.py:54-62)."""
    freqs = [theta ** (-2.0 * i / rotary_dim) for i in range(rotary_dim // 2)]
    if scaling is None:
        return freqs
    if scaling.rope_type != "llama3":
        raise ConfigError(f"rope scaling '{scaling.rope_type}' is not supported")
    orig = float(scaling.original_max_position_embeddings)
    lo, hi, factor = scaling.low_freq_factor, scaling.high_freq_factor, scaling.factor
    out = []
    for f in freqs:
        wavelen = 2.0 * math.pi / f
        if wavelen < orig / hi:
            out.append(f)
        elif wavelen > orig / lo:
            out.append(f / factor)
        else:
            s = (orig / wavelen - lo) / (hi - lo)
            out.append((1.0 - s) * f / factor + s * f)
    return out


@part("position", "rope")
class RotaryEmbedding(PositionEncoding):
    """Holds table[p] = (cos(p*f_0..), sin(p*f_0..)), [positions, rotary_dim] in 32-bit,
    computed in 64-bit and rounded once; it stands for the reference's stored ``rope``
    tensor (src/libllm/llama.cc:282-283)."""

    def __init__(self, spec, env):
        super().__init__(spec, env)
        if spec.rotary_dim % 2 or spec.rotary_dim > spec.head_dim or spec.rotary_dim <= 0:
            raise ConfigError(f"rotary width {spec.rotary_dim} does not fit head size {spec.head_dim}")
        self.table = None

    def load(self, fetch) -> None:
        spec, env = self.spec, self.env
        freqs = torch.tensor(rotary_frequencies(spec.rotary_dim, spec.theta, spec.scaling),
                             dtype=torch.float64, device=env.device)
        pos = torch.arange(env.max_positions, dtype=torch.float64, device=env.device)
        angle = pos[:, None] * freqs[None, :]
        self.table = torch.cat([angle.cos(), angle.sin()], dim=1).to(torch.float32).contiguous()
