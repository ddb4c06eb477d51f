"""Shared by the tests: the tiny configurations, model folders in temporary places, and
the comparison rule."""
from __future__ import annotations

import os
import tempfile
from typing import Dict, List

import torch

import plain_llama as P

# Two tiny configurations of the architecture that differ in every size and option.
TINY_A = dict(model_type="llama", num_hidden_layers=2, hidden_size=64, num_attention_heads=4,
              num_key_value_heads=2, head_dim=16, intermediate_size=192, vocab_size=256,
              rope_theta=10000.0, rope_scaling=None, rms_norm_eps=1e-5, tie_word_embeddings=True,
              max_position_embeddings=1024, eos_token_id=7, hidden_act="silu")
TINY_B = dict(model_type="llama", num_hidden_layers=3, hidden_size=96, num_attention_heads=3,
              num_key_value_heads=1, head_dim=32, intermediate_size=256, vocab_size=512,
              rope_theta=500000.0,
              rope_scaling=dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                                original_max_position_embeddings=64),
              rms_norm_eps=1e-6, tie_word_embeddings=False, max_position_embeddings=2048,
              eos_token_id=[3, 11], hidden_act="silu")
# A third one with sizes that are no power of two anywhere and a head size apart from hidden/heads.
TINY_C = dict(model_type="llama", num_hidden_layers=2, hidden_size=80, num_attention_heads=6,
              num_key_value_heads=3, head_dim=48, intermediate_size=176, vocab_size=331,
              rope_theta=50000.0, rope_scaling=None, rms_norm_eps=3e-6, tie_word_embeddings=False,
              max_position_embeddings=768, eos_token_id=None, hidden_act="silu")
TINY = {"A": TINY_A, "B": TINY_B, "C": TINY_C}

_folders: Dict[tuple, str] = {}
_tmp = None


def model_folder(name: str, seed: int = 1, config: dict = None) -> str:
    """A folder with config.json and model.safetensors (bfloat16) for a tiny configuration,
    made once per test session in a temporary place."""
    global _tmp
    key = (name, seed)
    if key not in _folders:
        from libllm_b200.weights import create_random_model
        if _tmp is None:
            _tmp = tempfile.TemporaryDirectory(prefix="libllm_b200_tests_")
        d = os.path.join(_tmp.name, f"{name}_{seed}")
        create_random_model(d, config or TINY[name], seed)
        _folders[key] = d
    return _folders[key]


def plain_weights(folder: str) -> Dict[str, torch.Tensor]:
    """The folder's tensors for the plain implementation, read without the library's loader."""
    import json
    import struct
    import numpy as np
    path = os.path.join(folder, "model.safetensors")
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        base = 8 + n
        blob = f.read()
    out = {}
    for name, e in header.items():
        if name == "__metadata__":
            continue
        b, end = e["data_offsets"]
        if e["dtype"] == "BF16":
            raw = np.frombuffer(blob[b:end], dtype=np.uint16).astype(np.uint32) << 16
            t = torch.from_numpy(raw.view(np.float32).copy())
        elif e["dtype"] == "F32":
            t = torch.from_numpy(np.frombuffer(blob[b:end], dtype=np.float32).copy())
        else:
            raise ValueError(e["dtype"])
        out[name] = t.reshape(e["shape"]).to(torch.float64)
    return out


def write_safetensors(path: str, tensors) -> None:
    """A safetensors file from a dict of torch tensors, written without the library."""
    import json
    import struct
    codes = {torch.float32: "F32", torch.float16: "F16", torch.bfloat16: "BF16", torch.float64: "F64", torch.int64: "I64",
             torch.int32: "I32", torch.uint8: "U8"}
    header, blobs, off = {}, [], 0
    for name, t in tensors.items():
        t = t.detach().cpu().contiguous()
        raw = (t.view(torch.int16) if t.dtype == torch.bfloat16 else t).numpy().tobytes()
        header[name] = dict(dtype=codes[t.dtype], shape=list(t.shape), data_offsets=[off, off + len(raw)])
        off += len(raw)
        blobs.append(raw)
    text = json.dumps(header).encode()
    text += b" " * ((8 - len(text) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(text)) + text + b"".join(blobs))


def rotary_frequencies(rotary_dim: int, theta: float, scaling):
    """The library's own frequencies (parts/builtin.cc), for tests that build a kernel's table."""
    import ctypes
    from libllm_b200 import _lib
    out = (ctypes.c_double * (rotary_dim // 2))()
    _lib.check(_lib.lib().llm_rotary_frequencies(rotary_dim, float(theta), _lib.Json(scaling).ref if scaling else _lib.Json(None).ref, out))
    return list(out)


def tokens_for(name: str, length: int, seed: int) -> List[int]:
    g = torch.Generator().manual_seed(1000 + seed)
    return torch.randint(0, TINY[name]["vocab_size"], (length,), generator=g).tolist()


def rel_err(got: torch.Tensor, ref: torch.Tensor) -> float:
    """max|got - ref| / mean|ref|, the reference's own measure (src/libllm/llama_test.cc:108-130)."""
    ref = ref.to(torch.float64)
    return float((got.to(torch.float64).cpu() - ref).abs().max() / ref.abs().mean())


def rms_err(got: torch.Tensor, ref: torch.Tensor) -> float:
    """||got - ref|| / ||ref||: unlike the maximum it is not set by one rare rounding."""
    ref = ref.to(torch.float64)
    d = got.to(torch.float64).cpu() - ref
    return float((d * d).mean().sqrt() / (ref * ref).mean().sqrt())


# Bounds: (on rel_err, on rms_err).
# float32: the engine and the plain implementation (float64) differ by 32-bit rounding alone.
# bfloat16: a bfloat16 matrix product takes bfloat16 inputs, so activations are rounded
#   (8 significant bits) at five places per layer and before the output matrix.  The plain
#   implementation itself, with these roundings and nothing else changed
#   (``forward_logits(..., act_dtype=torch.bfloat16)``), stands 1.0e-2 to 2.1e-2 (rel_err)
#   and 2e-3 to 4e-3 (rms_err) from its exact form on the tiny models here, and a
#   perturbation of 1e-7 before the roundings moves it by as much again, because
#   roundings flip and the flips spread: tests/test_plain.py measures both.  The bounds
#   are twice that floor.  (The reference allows 2e-2 in rel_err for float16, whose
#   rounding is eight times finer: src/libllm/llama_test.cc:49.)
TOL = {"float32": (2e-5, 2e-6), "bfloat16": (4e-2, 8e-3)}


def check_logits(got: torch.Tensor, ref: torch.Tensor, dtype: str, what: str = "") -> None:
    assert got.shape == ref.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(ref.shape)}"
    assert torch.isfinite(got).all(), f"{what}: logits are not finite"
    tol_max, tol_rms = TOL[dtype]
    e = rel_err(got, ref)
    assert e < tol_max, f"{what}: rel err {e:.3e} exceeds {tol_max:.1e} ({dtype})"
    r = rms_err(got, ref)
    assert r < tol_rms, f"{what}: rms err {r:.3e} exceeds {tol_rms:.1e} ({dtype})"
    # argmax agrees wherever the plain implementation's top-2 margin is above the tolerance
    ref64 = ref.to(torch.float64)
    if ref64.shape[-1] >= 2:
        top2 = ref64.topk(2, dim=-1).values
        margin = top2[..., 0] - top2[..., 1]
        clear = margin > 2 * tol_max * float(ref64.abs().mean())
        same = got.cpu().argmax(-1) == ref64.argmax(-1)
        assert bool((same | ~clear).all()), f"{what}: argmax differs where the margin is clear"


def check_against_plain(got: torch.Tensor, c: dict, w, toks, dtype: str, what: str = "") -> None:
    """The engine's logits for one whole request against the plain implementation."""
    import plain_llama as P
    check_logits(got, P.forward_logits(c, w, toks), dtype, what)
