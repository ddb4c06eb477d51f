"""The decode-attention entry point that allocates nothing, called through its exported C symbol.

``llm_attention_decode_static`` is for callers that cannot allocate device memory (a plug-in whose
host program owns all of it, a loop that may not stall on cudaMalloc): it joins the key splits
through an array built into the library instead of scratch the caller brings.  The test calls it
and the ordinary entry point (with scratch from torch) on the same inputs, twice in a row with
different lengths, so that what the first call left in the shared array is there when the second
runs, and compares the outputs.  This file is collected last on purpose: a run that stops at the
first failure has then run every other test."""
import ctypes
import math
from ctypes import c_float, c_int, c_longlong, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def library():
    from libllm_b200.csrc import build
    build.ensure_built(["attention_decode"])
    lib = ctypes.CDLL(build.library_path("attention_decode"))
    common = [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
              c_int, c_int, c_int, c_int, c_int, c_int, c_float]
    lib.llm_attention_decode.argtypes = common + [c_void_p, c_void_p, c_void_p]
    lib.llm_attention_decode_static.argtypes = common + [c_void_p]
    lib.llm_attention_decode.restype = lib.llm_attention_decode_static.restype = c_int
    lib.llm_attention_decode_last_error.restype = ctypes.c_char_p
    lib.llm_attention_decode_static_floats_needed.argtypes = [c_int, c_int, c_int, c_int]
    lib.llm_attention_decode_static_floats_needed.restype = c_longlong
    return lib


def make_inputs(lens, n_heads, n_kv, d, seed, page=64):
    g = torch.Generator().manual_seed(seed)
    B = len(lens)
    per = [(l + page - 1) // page for l in lens]
    n_pages = sum(per)
    perm = torch.randperm(n_pages, generator=g).tolist()
    table = torch.zeros((B, max(per)), dtype=torch.int32)
    o = 0
    for b in range(B):
        for j in range(per[b]):
            table[b, j] = perm[o]
            o += 1
    K = torch.randn((n_pages, n_kv, page, d), generator=g).to(torch.bfloat16).to(DEV)
    V = torch.randn((n_pages, n_kv, page, d), generator=g).to(torch.bfloat16).to(DEV)
    q = torch.randn((B, n_heads * d), generator=g).to(torch.bfloat16).to(DEV)
    pos = torch.tensor([l - 1 for l in lens], dtype=torch.int32, device=DEV)
    return q, K, V, table.to(DEV), pos


def call(lib, static, q, K, V, table, pos, n_heads, n_kv, d, chunk, n_splits):
    B = q.shape[0]
    out = torch.full((B, n_heads * d), float("nan"), dtype=torch.bfloat16, device=DEV)
    stream = c_void_p(torch.cuda.current_stream().cuda_stream)
    args = [c_void_p(q.data_ptr()), q.stride(0), c_void_p(out.data_ptr()), out.stride(0), c_void_p(K.data_ptr()),
            c_void_p(V.data_ptr()), c_void_p(pos.data_ptr()), c_void_p(table.data_ptr()), table.stride(0), B, n_heads,
            n_kv, d, 64, chunk, n_splits, 0, c_float(1.0 / math.sqrt(d))]
    if static:
        rc = lib.llm_attention_decode_static(*args, stream)
    else:
        ws_o = torch.full((B * n_heads * n_splits * d,), float("nan"), device=DEV)
        ws_ml = torch.full((B * n_heads * n_splits * 2,), float("nan"), device=DEV)
        rc = lib.llm_attention_decode(*args, c_void_p(ws_o.data_ptr()), c_void_p(ws_ml.data_ptr()), stream)
    torch.cuda.synchronize()
    return rc, out


def test_static_scratch_entry_point_matches_the_ordinary_one_twice_in_a_row():
    lib = library()
    n_heads, n_kv, d = 8, 2, 64
    for seed, lens, chunk, n_splits in ((1, [700, 64, 1, 333], 128, 6), (2, [65, 512, 40, 1000], 192, 6)):
        q, K, V, table, pos = make_inputs(lens, n_heads, n_kv, d, seed)
        rc0, want = call(lib, False, q, K, V, table, pos, n_heads, n_kv, d, chunk, n_splits)
        rc1, got = call(lib, True, q, K, V, table, pos, n_heads, n_kv, d, chunk, n_splits)
        assert rc0 == 0 and rc1 == 0, lib.llm_attention_decode_last_error()
        assert torch.isfinite(got.float()).all()
        err = float((got.float() - want.float()).abs().max())
        assert err <= 1e-2 * max(1.0, float(want.float().abs().max())), err      # the kernels tests' bound for bfloat16
        assert torch.equal(got, want)                                              # in fact the same kernels: the same bits


def test_static_scratch_entry_point_refuses_what_does_not_fit():
    lib = library()
    n_heads, n_kv, d = 32, 8, 128
    lens = [64] * 64
    q, K, V, table, pos = make_inputs(lens, n_heads, n_kv, d, 3)
    need = lib.llm_attention_decode_static_floats_needed(64, n_heads, d, 16)
    assert need == 64 * n_heads * 16 * (d + 2) and need > 2 * 1024 * 1024
    rc, _ = call(lib, True, q, K, V, table, pos, n_heads, n_kv, d, 64, 16)
    assert rc != 0
    msg = lib.llm_attention_decode_last_error().decode()
    assert "floats of scratch" in msg and str(need) in msg
    # one split needs no scratch at all and is taken at any size
    rc, out = call(lib, True, q, K, V, table, pos, n_heads, n_kv, d, 64, 1)
    assert rc == 0 and torch.isfinite(out.float()).all()
