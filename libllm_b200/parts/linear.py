"""y = x @ W^T (+ b) for the parts: picks the matrix product for the engine's type.

float32: the plain CUDA-core product with 32-bit accumulation (no tensor cores, no
reduced-precision mode).  bfloat16: the hand-written small-batch product when the step
has few tokens, the library product (cuBLAS through torch) otherwise, as the reference
calls cuBLAS for its products (src/flint/cuda/gemm_cublas.cc:160-197) and a kernel of
its own when one row is multiplied (src/flint/cuda/matvec.cu:61-87)."""
from __future__ import annotations

from typing import Optional

import torch

from ..csrc import ops
from ..errors import ExtensionError

_MM_OUT_DTYPE = None      # does torch.mm take out_dtype?  found out at the first call


def _library_mm(x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    global _MM_OUT_DTYPE
    if out_dtype == x.dtype:
        return torch.mm(x, w.t())
    if _MM_OUT_DTYPE is None:
        try:
            torch.mm(x[:1], w[:8].t(), out_dtype=out_dtype)
            _MM_OUT_DTYPE = True
        except (TypeError, RuntimeError):
            _MM_OUT_DTYPE = False
    if _MM_OUT_DTYPE:
        return torch.mm(x, w.t(), out_dtype=out_dtype)
    out = torch.empty((x.shape[0], w.shape[0]), dtype=out_dtype, device=x.device)
    return ops.gemm_plain(x, w, out)


def linear(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None,
           out_dtype: Optional[torch.dtype] = None, parts_ok: bool = False) -> torch.Tensor:
    """x [T, K] in the engine's type, w [N, K]; returns [T, N] in ``out_dtype``.  With
    ``parts_ok`` (for results that go into the residual addition, which adds parts in
    order) the result may be [parts, T, N] partial products to be summed."""
    if not x.is_cuda:
        raise ExtensionError("linear: activations must be on a CUDA device (there is no CPU fallback)")
    out_dtype = out_dtype or x.dtype
    T = x.shape[0]
    if x.dtype == torch.float32 or bias is not None:
        out = torch.empty((T, w.shape[0]), dtype=out_dtype, device=x.device)
        return ops.gemm_plain(x, w, out, bias)
    from . import fast
    y = fast.small_batch_linear(x, w, out_dtype, parts_ok=parts_ok)
    if y is not None:
        return y
    return _library_mm(x, w, out_dtype)
