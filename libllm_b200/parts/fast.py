"""Switchboard of the fast bfloat16 kernels: each entry returns None when the kernel
does not take the case, and the caller then uses the general kernel.  Kernels are
switched on one at a time as they pass their tests."""
from __future__ import annotations

import os
from typing import Optional

import torch

ENABLED = {
    "gemv": os.environ.get("LIBLLM_B200_NO_GEMV") is None,
    "decode_attention": os.environ.get("LIBLLM_B200_NO_DECODE_ATTENTION") is None,
    "prefill_attention": os.environ.get("LIBLLM_B200_NO_PREFILL_ATTENTION") is None,
}


def small_batch_linear(x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype) -> Optional[torch.Tensor]:
    return None


def attention(ctx, qkv: torch.Tensor, cache, spec, scale: float) -> Optional[torch.Tensor]:
    return None
