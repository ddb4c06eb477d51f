"""Python faces of the CUDA kernels: each takes torch tensors on a CUDA device, checks
what the kernel relies on (device, type, contiguity, alignment) and launches on the
current stream.  Nothing here computes on the host or falls back to torch operators:
a tensor that is not on a CUDA device is an error."""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Optional

import torch

from ..errors import ExtensionError, UnsupportedError
from . import build

F32, BF16 = 0, 1
_DT = {torch.float32: F32, torch.bfloat16: BF16}


def dtype_code(dt: torch.dtype) -> int:
    try:
        return _DT[dt]
    except KeyError:
        raise UnsupportedError(f"element type {dt} is not supported (float32 or bfloat16)") from None


def _ptr(t: Optional[torch.Tensor]) -> c_void_p:
    return c_void_p(0 if t is None else t.data_ptr())


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> c_void_p:
    """The current stream's handle.  Asked for at every launch, so by the short way where torch has
    one (building a Stream object costs more than the launch itself)."""
    if _raw_stream is not None:
        return c_void_p(_raw_stream(torch.cuda.current_device()))
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _on_gpu(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise ExtensionError("libllm_b200 kernels run on a CUDA device only; got a tensor on "
                                 f"'{t.device}' (there is no CPU fallback)")


_protos = {}
LAUNCHES = [0]        # kernel launches issued through this module (graph replays not included)


def _fn(family: str, name: str, argtypes):
    key = (family, name)
    f = _protos.get(key)
    if f is None:
        lib = build.load(family)
        f = getattr(lib, name)
        f.argtypes = argtypes
        f.restype = c_int
        err = getattr(lib, f"llm_{family}_last_error")
        err.restype = ctypes.c_char_p
        _protos[key] = f = (f, err)
    return f


def _call(family: str, name: str, argtypes, *args) -> None:
    f, err = _fn(family, name, argtypes)
    LAUNCHES[0] += 1
    status = f(*args)
    if status != 0:
        msg = err().decode("utf-8", "replace")
        if status == 0x0100:
            raise UnsupportedError(msg)
        raise ExtensionError(f"{name} failed (status {status:#x}): {msg}")


# ------------------------------------------------------------------ elementwise
def embedding(table: torch.Tensor, tokens: torch.Tensor, out: torch.Tensor,
              fed_tokens: Optional[torch.Tensor] = None, fed_rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[t, :] = float(table[id_t, :]); out is the 32-bit residual stream.  id_t is tokens[t], or,
    where fed_rows[t] >= 0, fed_tokens[fed_rows[t]]: a token the previous step left on the device."""
    _on_gpu(table, tokens, out, fed_tokens, fed_rows)
    n = tokens.numel()
    assert tokens.dtype == torch.int32 and out.dtype == torch.float32
    assert table.is_contiguous() and out.is_contiguous() and tuple(out.shape) == (n, table.shape[1])
    if fed_rows is not None:
        assert fed_tokens is not None and fed_tokens.dtype == torch.int32 and fed_rows.dtype == torch.int32
        assert fed_rows.numel() >= n
    _call("elementwise", "llm_embedding",
          [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
          dtype_code(table.dtype), _ptr(table), _ptr(tokens), _ptr(fed_tokens if fed_rows is not None else None),
          _ptr(fed_rows), _ptr(out), n, table.shape[1], table.shape[0], _stream())
    return out


def copy_words(src: torch.Tensor, dst: torch.Tensor, n: int) -> None:
    """n 32-bit words from src to dst by a kernel; one of the two may be pinned host memory."""
    assert src.dtype == torch.int32 and dst.dtype == torch.int32 and src.numel() >= n and dst.numel() >= n
    assert src.is_contiguous() and dst.is_contiguous()
    for t in (src, dst):
        if not (t.is_cuda or t.is_pinned()):
            raise ExtensionError("copy_words: host memory must be pinned")
    _call("elementwise", "llm_copy_words", [c_void_p, c_void_p, c_int, c_void_p], _ptr(src), _ptr(dst), int(n), _stream())


def add_rmsnorm(resid: torch.Tensor, delta: Optional[torch.Tensor], weight: Optional[torch.Tensor],
                eps: float, out: Optional[torch.Tensor], rows: Optional[torch.Tensor] = None) -> None:
    """resid += sum of delta's parts (32-bit, written back unless ``rows`` selects a
    subset), then out = rmsnorm(resid) * weight.  ``delta`` is [T, H] or [parts, T, H]."""
    _on_gpu(resid, delta, weight, out, rows)
    assert resid.dtype == torch.float32 and resid.is_contiguous() and resid.dim() == 2
    T, H = resid.shape
    n_parts, stride, ddt = 0, 0, F32
    if delta is not None:
        assert delta.is_contiguous() and delta.shape[-2:] == resid.shape
        n_parts = 1 if delta.dim() == 2 else delta.shape[0]
        stride = T * H
        ddt = dtype_code(delta.dtype)
    n_rows = T if rows is None else rows.numel()
    odt = F32
    if out is not None:
        assert weight is not None and weight.dtype == torch.float32 and weight.numel() == H
        assert out.is_contiguous() and tuple(out.shape) == (n_rows, H)
        odt = dtype_code(out.dtype)
    if rows is not None:
        assert rows.dtype == torch.int32
    _call("elementwise", "llm_add_rmsnorm",
          [c_void_p, c_void_p, c_int, c_int, c_longlong, c_void_p, c_float, c_void_p, c_int, c_void_p,
           c_int, c_int, c_void_p],
          _ptr(resid), _ptr(delta), ddt, n_parts, stride, _ptr(weight), float(eps), _ptr(out), odt,
          _ptr(rows), n_rows, H, _stream())


def swiglu(gu: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[t, i] = silu(gu[t, i]) * gu[t, I + i]; gu may be 32-bit while out is bfloat16."""
    _on_gpu(gu, out)
    T, two_i = gu.shape
    assert gu.is_contiguous() and out.is_contiguous()
    assert tuple(out.shape) == (T, two_i // 2)
    _call("elementwise", "llm_swiglu", [c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_void_p],
          dtype_code(gu.dtype), dtype_code(out.dtype), _ptr(gu), _ptr(out), T, two_i // 2, _stream())
    return out


# ------------------------------------------------------------------ plain matrix product
def gemm_plain(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor,
               bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[M, N] = a[M, K] @ w[N, K]^T (+ bias) on the CUDA cores, 32-bit accumulate."""
    _on_gpu(a, w, out, bias)
    M, K = a.shape
    N = w.shape[0]
    assert w.shape[1] == K and tuple(out.shape) == (M, N)
    assert a.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1 and a.dtype == w.dtype
    if bias is not None:
        assert bias.dtype == torch.float32 and bias.numel() == N
    _call("gemm_plain", "llm_gemm_plain",
          [c_int, c_int, c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_void_p, c_longlong,
           c_int, c_int, c_int, c_void_p],
          dtype_code(a.dtype), dtype_code(out.dtype), _ptr(a), a.stride(0) if M > 1 else K, _ptr(w),
          w.stride(0), _ptr(bias), _ptr(out), out.stride(0) if M > 1 else N, M, N, K, _stream())
    return out


# ------------------------------------------------------------------ rope + cache write
def rope_cache_write(qkv: torch.Tensor, q_out: torch.Tensor, n_heads: int, n_kv: int, head_dim: int,
                     table: torch.Tensor, tok_seq: torch.Tensor, tok_pos: torch.Tensor,
                     page_table: torch.Tensor, kcache: Optional[torch.Tensor],
                     vcache: Optional[torch.Tensor], page_size: int, write_cache: bool = True) -> None:
    """Rotates the q heads of the stacked rows into ``q_out`` and, rotated (k) or as they
    are (v), appends k and v to the paged cache [pages, kv_heads, page_size, d] of one
    layer.  ``qkv`` may be 32-bit while ``q_out`` and the cache are bfloat16."""
    _on_gpu(qkv, q_out, table, tok_seq, tok_pos, page_table, kcache, vcache)
    T = qkv.shape[0]
    assert qkv.stride(1) == 1 and qkv.shape[1] == (n_heads + 2 * n_kv) * head_dim
    assert q_out.stride(1) == 1 and q_out.shape[0] == T and q_out.shape[1] >= n_heads * head_dim
    assert table.dtype == torch.float32 and table.is_contiguous() and table.dim() == 2
    assert page_table.dtype == torch.int32 and page_table.dim() == 2 and page_table.stride(1) == 1
    if write_cache:
        assert kcache.dtype == q_out.dtype and kcache.is_contiguous() and vcache.is_contiguous()
        assert tuple(kcache.shape[1:]) == (n_kv, page_size, head_dim)
    _call("rope", "llm_rope_cache_write",
          [c_int, c_int, c_void_p, c_longlong, c_void_p, c_longlong, c_int, c_int, c_int, c_int, c_void_p,
           c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_void_p],
          dtype_code(qkv.dtype), dtype_code(q_out.dtype), _ptr(qkv), qkv.stride(0), _ptr(q_out),
          q_out.stride(0), T, n_heads, n_kv, head_dim, _ptr(table), table.shape[0], table.shape[1],
          _ptr(tok_seq), _ptr(tok_pos), _ptr(page_table), page_table.stride(0), _ptr(kcache), _ptr(vcache),
          page_size, 1 if write_cache else 0, _stream())


# ------------------------------------------------------------------ attention (generic)
def attention_generic(q: torch.Tensor, out: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor,
                      tok_seq: torch.Tensor, tok_pos: torch.Tensor, page_table: torch.Tensor,
                      n_heads: int, n_kv: int, head_dim: int, page_size: int, window: Optional[int],
                      scale: float) -> torch.Tensor:
    """q is a [T, >= n_heads*d] view whose first n_heads*d columns are the rotated queries."""
    _on_gpu(q, out, kcache, vcache, tok_seq, tok_pos, page_table)
    T = q.shape[0]
    assert q.stride(1) == 1 and out.stride(1) == 1 and out.shape[0] == T and out.shape[1] == n_heads * head_dim
    assert kcache.dtype == q.dtype and out.dtype == q.dtype
    _call("attention_generic", "llm_attention_generic",
          [c_int, c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p,
           c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p],
          dtype_code(q.dtype), _ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(kcache), _ptr(vcache),
          _ptr(tok_seq), _ptr(tok_pos), _ptr(page_table), page_table.stride(0), T, n_heads, n_kv, head_dim,
          page_size, int(window or 0), float(scale), _stream())
    return out


# ------------------------------------------------------------------ sampling
def argmax(logits: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    _on_gpu(logits, out)
    assert logits.dtype == torch.float32 and logits.stride(1) == 1 and out.dtype == torch.int32
    _call("sampling", "llm_argmax", [c_void_p, c_longlong, c_int, c_int, c_void_p, c_void_p],
          _ptr(logits), logits.stride(0), logits.shape[0], logits.shape[1], _ptr(out), _stream())
    return out


def sample(logits: torch.Tensor, temperature: float, top_k: int, top_p: float, uniforms: torch.Tensor,
           out: torch.Tensor) -> torch.Tensor:
    _on_gpu(logits, uniforms, out)
    assert logits.dtype == torch.float32 and logits.stride(1) == 1 and out.dtype == torch.int32
    assert uniforms.dtype == torch.float32 and uniforms.numel() >= logits.shape[0]
    _call("sampling", "llm_sample",
          [c_void_p, c_longlong, c_int, c_int, c_float, c_int, c_float, c_void_p, c_void_p, c_void_p],
          _ptr(logits), logits.stride(0), logits.shape[0], logits.shape[1], float(temperature), int(top_k),
          float(top_p), _ptr(uniforms), _ptr(out), _stream())
    return out


# ------------------------------------------------------------------ small-batch product (bfloat16)
GEMV_MAX_TOKENS = 64


def gemv_supported(x: torch.Tensor, w: torch.Tensor) -> bool:
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and 0 < x.shape[0] <= GEMV_MAX_TOKENS
            and x.shape[1] % 8 == 0 and x.stride(1) == 1 and x.stride(0) % 8 == 0 and w.is_contiguous()
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gemv_suggest_parts(M: int, N: int, K: int) -> int:
    lib = build.load("gemv")
    f = lib.llm_gemv_suggest_parts
    f.argtypes, f.restype = [c_int, c_int, c_int], c_int
    return int(f(M, N, K))


def gemv_bf16(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, swiglu: bool = False) -> torch.Tensor:
    """out[M, N] = x[M, K] @ w[N, K]^T for M <= 64; with ``swiglu`` w is the stacked
    gate|up matrix [2I, K] and out[M, I] = silu(gate) * up.  A 3-d ``out`` [parts, M, N]
    (32-bit) receives partial products over parts of K, to be added by the caller."""
    _on_gpu(x, w, out)
    M, K = x.shape
    N = w.shape[0]
    parts, stride = 1, 0
    if out.dim() == 3:
        parts, stride = out.shape[0], out.stride(0)
        assert out.dtype == torch.float32 and not swiglu and out.is_contiguous()
    assert w.shape[1] == K and out.stride(-1) == 1 and tuple(out.shape[-2:]) == (M, N // 2 if swiglu else N)
    _call("gemv", "llm_gemv_bf16",
          [c_void_p, c_longlong, c_void_p, c_void_p, c_longlong, c_int, c_int, c_int, c_int, c_int, c_int,
           c_longlong, c_void_p],
          _ptr(x), x.stride(0) if M > 1 else K, _ptr(w), _ptr(out), out.stride(-2) if M > 1 else out.shape[-1],
          dtype_code(out.dtype), M, N, K, 1 if swiglu else 0, parts, stride, _stream())
    return out


# ------------------------------------------------------------------ attention for decoding (bfloat16)
def attention_decode_supported(head_dim: int, group: int) -> bool:
    lib = build.load("attention_decode")
    f = lib.llm_attention_decode_supports
    f.argtypes, f.restype = [c_int, c_int], c_int
    return bool(f(head_dim, group))


def attention_decode(q: torch.Tensor, out: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor,
                     tok_pos: torch.Tensor, page_table: torch.Tensor, n_heads: int, n_kv: int, head_dim: int,
                     page_size: int, chunk: int, n_splits: int, window: Optional[int], scale: float,
                     ws_o: Optional[torch.Tensor], ws_ml: Optional[torch.Tensor]) -> torch.Tensor:
    """One query token per sequence over the paged cache, keys split into ``n_splits``
    runs of ``chunk``; ``ws_o``/``ws_ml`` are the scratch the splits are joined through."""
    _on_gpu(q, out, kcache, vcache, tok_pos, page_table, ws_o, ws_ml)
    B = q.shape[0]
    assert q.dtype == torch.bfloat16 and kcache.dtype == torch.bfloat16 and out.dtype == torch.bfloat16
    assert q.stride(1) == 1 and out.stride(1) == 1 and tok_pos.numel() >= B
    if n_splits > 1:
        assert ws_o.dtype == torch.float32 and ws_o.numel() >= B * n_heads * n_splits * head_dim
        assert ws_ml.dtype == torch.float32 and ws_ml.numel() >= B * n_heads * n_splits * 2
    _call("attention_decode", "llm_attention_decode",
          [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
           c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p, c_void_p, c_void_p],
          _ptr(q), q.stride(0) if B > 1 else q.shape[1], _ptr(out), out.stride(0) if B > 1 else out.shape[1],
          _ptr(kcache), _ptr(vcache), _ptr(tok_pos), _ptr(page_table), page_table.stride(0), B, n_heads, n_kv,
          head_dim, page_size, chunk, n_splits, int(window or 0), float(scale), _ptr(ws_o), _ptr(ws_ml), _stream())
    return out


# ------------------------------------------------------------------ attention for prompts (bfloat16)
def attention_prefill_supported(head_dim: int, page_size: int) -> bool:
    lib = build.load("attention_prefill")
    f = lib.llm_attention_prefill_supports
    f.argtypes, f.restype = [c_int, c_int], c_int
    return bool(f(head_dim, page_size))


def attention_prefill(q: torch.Tensor, out: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor,
                      seq_start: torch.Tensor, seq_past: torch.Tensor, page_table: torch.Tensor, n_seqs: int,
                      max_q_len: int, n_heads: int, n_kv: int, head_dim: int, page_size: int,
                      window: Optional[int], scale: float) -> torch.Tensor:
    """Causal attention of every sequence's new tokens (rows seq_start[b]..seq_start[b+1]-1 of
    ``q``, standing behind seq_past[b] cached tokens) over the paged cache, which already
    holds the new tokens' keys and values."""
    _on_gpu(q, out, kcache, vcache, seq_start, seq_past, page_table)
    assert q.dtype == torch.bfloat16 and kcache.dtype == torch.bfloat16 and out.dtype == torch.bfloat16
    assert q.stride(1) == 1 and out.stride(1) == 1 and out.shape[0] == q.shape[0]
    assert seq_start.dtype == torch.int32 and seq_past.dtype == torch.int32 and page_table.dtype == torch.int32
    assert seq_start.numel() >= n_seqs + 1 and seq_past.numel() >= n_seqs and page_table.shape[0] >= n_seqs
    assert kcache.is_contiguous() and vcache.is_contiguous()
    assert tuple(kcache.shape[1:]) == (n_kv, page_size, head_dim)
    _call("attention_prefill", "llm_attention_prefill",
          [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
           c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p],
          _ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(kcache), _ptr(vcache), _ptr(seq_start),
          _ptr(seq_past), _ptr(page_table), page_table.stride(0), n_seqs, max_q_len, n_heads, n_kv, head_dim,
          page_size, int(window or 0), float(scale), _stream())
    return out


# ------------------------------------------------------------------ product on tcgen05 tensor cores (bfloat16)
_tc_status = {}


def tc_status(device) -> torch.Tensor:
    """The device word in which the tensor-core kernels record that a wait ran out of time."""
    dev = torch.device(device)
    t = _tc_status.get(dev)
    if t is None:
        t = _tc_status[dev] = torch.zeros(1, dtype=torch.int32, device=dev)
    return t


def check_tc_status() -> None:
    """Raises if a tensor-core kernel gave up waiting since the last check (this reads the word
    back, so it waits for the device)."""
    for dev, t in _tc_status.items():
        code = int(t.item())
        if code:
            t.zero_()
            raise ExtensionError(f"a tensor-core kernel on {dev} gave up waiting on a barrier (code {code}: "
                                 "1 loader, 2-3 issue, 4-6 epilogue); its results are not valid")


def gemm_tc_supported(x: torch.Tensor, w: torch.Tensor) -> bool:
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.shape[0] > 0 and x.shape[1] % 8 == 0
            and x.stride(1) == 1 and (x.shape[0] == 1 or x.stride(0) % 8 == 0) and w.is_contiguous()
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gemm_tc_suggest_parts(M: int, N: int, K: int) -> int:
    lib = build.load("gemm_tc")
    f = lib.llm_gemm_tc_suggest_parts
    f.argtypes, f.restype = [c_int, c_int, c_int], c_int
    return int(f(M, N, K))


def gemm_tc(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, swiglu: bool = False) -> torch.Tensor:
    """out[M, N] = x[M, K] @ w[N, K]^T on tcgen05 with TMA-fed operands, for any M; with ``swiglu`` w
    is the stacked gate|up matrix [2I, K] and out[M, I] = silu(gate) * up.  A 3-d ``out``
    [parts, M, N] (32-bit) receives partial products over parts of K, to be added by the caller."""
    _on_gpu(x, w, out)
    M, K = x.shape
    N = w.shape[0]
    parts, stride = 1, 0
    if out.dim() == 3:
        parts, stride = out.shape[0], out.stride(0)
        assert out.dtype == torch.float32 and not swiglu and out.is_contiguous()
    assert w.shape[1] == K and out.stride(-1) == 1 and tuple(out.shape[-2:]) == (M, N // 2 if swiglu else N)
    _call("gemm_tc", "llm_gemm_tc",
          [c_void_p, c_longlong, c_void_p, c_void_p, c_longlong, c_int, c_int, c_int, c_int, c_int, c_int,
           c_longlong, c_void_p, c_void_p],
          _ptr(x), x.stride(0) if M > 1 else K, _ptr(w), _ptr(out), out.stride(-2) if M > 1 else out.shape[-1],
          dtype_code(out.dtype), M, N, K, 1 if swiglu else 0, parts, stride, _ptr(tc_status(x.device)), _stream())
    return out


# ------------------------------------------------------------------ a chain of products and norms in one launch
class ChainJob(ctypes.Structure):
    """The kernel library's llm_chain_job (libllm_b200/csrc/gemm_chain.cu)."""
    _fields_ = [("kind", c_int), ("dep0", c_int), ("dep1", c_int), ("x", c_void_p), ("ldx", c_longlong),
                ("w", c_void_p), ("out", c_void_p), ("ldo", c_longlong), ("M", c_int), ("N", c_int), ("K", c_int),
                ("k_parts", c_int), ("part_stride", c_longlong), ("resid", c_void_p), ("delta", c_void_p),
                ("delta_parts", c_int), ("delta_stride", c_longlong), ("weight", c_void_p), ("eps", ctypes.c_float),
                ("rows", c_void_p), ("n_rows", c_int), ("hidden", c_int)]


def chain_product(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, swiglu: bool = False, deps=(-1, -1)) -> ChainJob:
    """A product job: out [M, N] or [parts, M, N] 32-bit, or with ``swiglu`` [M, N/2] bfloat16."""
    _on_gpu(x, w, out)
    M, K = x.shape
    j = ChainJob()
    j.kind, j.dep0, j.dep1 = (1 if swiglu else 0), deps[0], deps[1]
    j.x, j.ldx, j.w, j.out = _ptr(x), (x.stride(0) if M > 1 else K), _ptr(w), _ptr(out)
    j.ldo = out.stride(-2) if M > 1 else out.shape[-1]
    j.M, j.N, j.K = M, w.shape[0], K
    j.k_parts, j.part_stride = (out.shape[0], out.stride(0)) if out.dim() == 3 else (1, 0)
    return j


def chain_norm(resid: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float, out: torch.Tensor,
               rows: Optional[torch.Tensor] = None, deps=(-1, -1)) -> ChainJob:
    """An add + RMSNorm job: delta [parts, T, H] or [T, H] 32-bit is added to resid [T, H] first."""
    j = ChainJob()
    j.kind, j.dep0, j.dep1 = 2, deps[0], deps[1]
    j.resid, j.weight, j.out, j.eps = _ptr(resid), _ptr(weight), _ptr(out), eps
    if delta is not None:
        j.delta = _ptr(delta)
        j.delta_parts, j.delta_stride = (delta.shape[0], delta.stride(0)) if delta.dim() == 3 else (1, 0)
    j.rows = _ptr(rows)
    j.n_rows, j.hidden = out.shape[0], resid.shape[1]
    return j


def gemm_chain(jobs, counters: torch.Tensor) -> None:
    """Runs the jobs in order as one launch; ``counters`` are at least 9 int32 zeros, left zero."""
    arr = (ChainJob * len(jobs))(*jobs)
    _call("gemm_chain", "llm_gemm_chain", [c_void_p, c_int, c_void_p, c_void_p, c_void_p],
          ctypes.cast(arr, c_void_p), len(jobs), _ptr(counters), _ptr(tc_status(counters.device)), _stream())


# ------------------------------------------------------------------ decode attention on tensor cores, rotation fused
def attention_decode_tc_supported(head_dim: int, page_size: int, group: int) -> bool:
    lib = build.load("attention_decode_tc")
    f = lib.llm_attention_decode_tc_supports
    f.argtypes, f.restype = [c_int, c_int, c_int], c_int
    return bool(f(head_dim, page_size, group))


def attention_decode_tc_ctas_per_sm(head_dim: int) -> int:
    lib = build.load("attention_decode_tc")
    f = lib.llm_attention_decode_tc_ctas_per_sm
    f.argtypes, f.restype = [c_int], c_int
    return int(f(head_dim))


def attention_decode_tc(qkv: torch.Tensor, out: torch.Tensor, table: torch.Tensor, kcache: torch.Tensor,
                        vcache: torch.Tensor, tok_pos: torch.Tensor, page_table: torch.Tensor, n_heads: int,
                        n_kv: int, head_dim: int, page_size: int, chunk: int, n_splits: int, window: Optional[int],
                        scale: float, write_cache: bool, ws_o: Optional[torch.Tensor],
                        ws_ml: Optional[torch.Tensor], counters: Optional[torch.Tensor],
                        max_len: int = 0) -> torch.Tensor:
    """One token per sequence: rotates q and k of the 32-bit stacked rows ``qkv``, appends k and v to
    the cache (with ``write_cache``), attends over the cache and joins the key splits, in one launch.
    ``counters`` (int32, one per sequence and kv head) must be zero before the first launch; the
    kernel leaves it zero.  ``chunk`` 0 cuts each sequence's own length into ``n_splits`` runs; ``max_len``
    then bounds the lengths."""
    _on_gpu(qkv, out, table, kcache, vcache, tok_pos, page_table, ws_o, ws_ml, counters)
    parts, part_stride = 1, 0
    if qkv.dim() == 3:                       # [parts, B, W]: partial products over K, added in the kernel
        parts, part_stride = qkv.shape[0], qkv.stride(0)
        qkv2 = qkv[0]
    else:
        qkv2 = qkv
    B = qkv2.shape[0]
    assert qkv.dtype == torch.float32 and qkv2.dim() == 2 and qkv2.stride(1) == 1
    assert qkv2.shape[1] == (n_heads + 2 * n_kv) * head_dim
    assert kcache.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and out.stride(1) == 1
    assert kcache.is_contiguous() and vcache.is_contiguous() and tuple(kcache.shape[1:]) == (n_kv, page_size, head_dim)
    assert table.dtype == torch.float32 and table.is_contiguous() and table.dim() == 2
    assert tok_pos.dtype == torch.int32 and tok_pos.numel() >= B and page_table.dtype == torch.int32
    if n_splits > 1:
        assert ws_o.dtype == torch.float32 and ws_o.numel() >= B * n_heads * n_splits * head_dim
        assert ws_ml.dtype == torch.float32 and ws_ml.numel() >= B * n_heads * n_splits * 2
        assert counters.dtype == torch.int32 and counters.numel() >= B * n_kv
    _call("attention_decode_tc", "llm_attention_decode_tc",
          [c_void_p, c_longlong, c_int, c_longlong, c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p,
           c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p, c_void_p,
           c_void_p, c_void_p, c_longlong, c_void_p],
          _ptr(qkv), qkv2.stride(0) if B > 1 else qkv2.shape[1], parts, part_stride, _ptr(table), table.shape[0],
          table.shape[1],
          _ptr(tok_pos), _ptr(page_table), page_table.stride(0), _ptr(kcache), _ptr(vcache), 1 if write_cache else 0,
          B, n_heads, n_kv, head_dim, page_size, chunk, int(max_len), n_splits, int(window or 0), float(scale),
          _ptr(ws_o), _ptr(ws_ml), _ptr(counters), _ptr(out), out.stride(0) if B > 1 else out.shape[1], _stream())
    return out


# ------------------------------------------------------------------ attention for prompts on tcgen05 (bfloat16)
def attention_prefill_tc_supported(head_dim: int, page_size: int) -> bool:
    lib = build.load("attention_prefill_tc")
    f = lib.llm_attention_prefill_tc_supports
    f.argtypes, f.restype = [c_int, c_int], c_int
    return bool(f(head_dim, page_size))


def attention_prefill_tc(q: torch.Tensor, out: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor,
                         seq_start: torch.Tensor, seq_past: torch.Tensor, page_table: torch.Tensor, n_seqs: int,
                         max_q_len: int, n_heads: int, n_kv: int, head_dim: int, page_size: int,
                         window: Optional[int], scale: float, form: int = 0) -> torch.Tensor:
    """The same attention as ``attention_prefill`` with both products on tcgen05 (head sizes 64, 128).
    ``form``: 1 for CTAs of 128 query rows and tiles of 64 keys, 2 for CTAs of 256 rows and tiles of
    128 keys, 0 for the library's choice (the second when a sequence brings more than 128 rows)."""
    _on_gpu(q, out, kcache, vcache, seq_start, seq_past, page_table)
    assert q.dtype == torch.bfloat16 and kcache.dtype == torch.bfloat16 and out.dtype == torch.bfloat16
    assert q.stride(1) == 1 and out.stride(1) == 1 and out.shape[0] == q.shape[0]
    assert seq_start.dtype == torch.int32 and seq_past.dtype == torch.int32 and page_table.dtype == torch.int32
    assert kcache.is_contiguous() and vcache.is_contiguous() and tuple(kcache.shape[1:]) == (n_kv, page_size, head_dim)
    _call("attention_prefill_tc", "llm_attention_prefill_tc",
          [c_void_p, c_longlong, c_longlong, c_void_p, c_longlong, c_void_p, c_void_p, c_longlong, c_void_p, c_void_p,
           c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p, c_void_p],
          _ptr(q), q.stride(0), q.shape[0], _ptr(out), out.stride(0), _ptr(kcache), _ptr(vcache), kcache.shape[0],
          _ptr(seq_start), _ptr(seq_past), _ptr(page_table), page_table.stride(0), n_seqs, max_q_len, n_heads, n_kv,
          head_dim, page_size, int(window or 0), float(scale), int(form), _ptr(tc_status(q.device)), _stream())
    return out
