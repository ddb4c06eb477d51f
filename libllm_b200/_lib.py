"""ctypes face of the host library (include/llm.h): loading, JSON handles, and the mapping from a
status to this package's exceptions.  Everything else in the Python package goes through here;
nothing in Python computes, loads weights or keeps a cache of its own."""
from __future__ import annotations

import ctypes
import json
from ctypes import (POINTER, c_char_p, c_double, c_float, c_int32, c_int64, c_uint64, c_void_p)
from typing import Any, List, Optional, Sequence

from . import errors
from .csrc import build

_lib = None
_registered = set()

_KINDS = {1: errors.InvalidArgError, 2: errors.ConfigError, 3: errors.WeightsError, 4: errors.CacheError,
          5: errors.UnsupportedError, 6: errors.ExtensionError, 7: errors.LlmError, 8: errors.EndOfSequence}


def lib() -> ctypes.CDLL:
    """The host library, built on first use."""
    global _lib
    if _lib is None:
        L = build.load_host()
        P = c_void_p
        PP = POINTER(c_void_p)
        I32P, I64P, F32P = POINTER(c_int32), POINTER(c_int64), POINTER(c_float)
        sigs = {
            "llm_get_last_error_message": (c_char_p, []),
            "llm_get_last_error_kind": (c_int32, []),
            "llm_get_last_error_details": (c_char_p, []),
            "llm_json_init": (c_int32, [PP]), "llm_json_destroy": (c_int32, [PP]),
            "llm_json_parse": (c_int32, [PP, c_char_p]), "llm_json_dump": (c_int32, [PP, c_char_p, c_int64]),
            "llm_json_dump_size": (c_int64, [PP]),
            "llm_model_init": (c_int32, [PP]), "llm_model_destroy": (c_int32, [PP]),
            "llm_model_load": (c_int32, [PP, PP]), "llm_model_get_info": (c_int32, [PP, PP]),
            "llm_model_complete": (c_int32, [PP, PP, PP]),
            "llm_completion_init": (c_int32, [PP]), "llm_completion_destroy": (c_int32, [PP]),
            "llm_completion_get_next_chunk": (c_int32, [PP, PP]),
            "llm_model_load_tensors": (c_int32, [PP, PP, c_int32, POINTER(c_char_p), POINTER(c_char_p), POINTER(I64P), I32P,
                                                 POINTER(c_void_p)]),
            "llm_model_generate": (c_int32, [PP, PP, c_void_p, c_void_p, PP]),
            "llm_model_open_sequence": (c_int32, [PP, I32P]), "llm_model_close_sequence": (c_int32, [PP, c_int32]),
            "llm_model_sequence_length": (c_int32, [PP, c_int32, I32P]),
            "llm_model_step": (c_int32, [PP, c_int32, I32P, I32P, I32P, I32P, I32P, I32P, c_char_p, F32P, F32P, I32P]),
            "llm_model_step_tokens": (c_int32, [PP, c_int32, I32P, I32P, I32P, I32P, I32P, c_char_p, F32P, PP]),
            "llm_pending_result": (c_int32, [PP, I32P]), "llm_pending_destroy": (c_int32, [PP]),
            "llm_model_synchronize": (c_int32, [PP]), "llm_model_stream": (c_int32, [PP, PP]),
            "llm_model_cache_info": (c_int32, [PP, PP]), "llm_model_cache_check": (c_int32, [PP]),
            "llm_model_debug_set_status": (c_int32, [PP, c_int32]), "llm_model_debug_wait_probe": (c_int32, [PP, c_int64]),
            "llm_known_architectures": (c_int32, [PP]), "llm_load_config": (c_int32, [c_char_p, PP]),
            "llm_parse_config": (c_int32, [PP, PP]), "llm_describe_model": (c_int32, [PP, c_char_p, PP]),
            "llm_create_random_model": (c_int32, [c_char_p, PP, c_uint64, c_char_p]),
            "llm_check_weights": (c_int32, [c_char_p, PP, PP, c_int32, PP]),
            "llm_read_safetensors_header": (c_int32, [c_char_p, PP]),
            "llm_set_kernel_library": (c_int32, [c_char_p, c_char_p]), "llm_loaded_kernel_libraries": (c_int32, [PP]),
            "llm_kernel_launches": (c_int64, []),
            "llm_rotary_frequencies": (c_int32, [c_int64, c_double, PP, POINTER(c_double)]),
            "llm_uniform": (c_float, [c_uint64, c_uint64, c_uint64]),
            "llm_plan_batches": (c_int32, [PP, PP]), "llm_validate_sampling": (c_int32, [c_double, c_int32, c_double]),
            "llm_should_stop": (c_int32, [c_int32, c_int32, c_int32, PP, PP]),
            "llm_cachebook_init": (c_int32, [PP, PP]), "llm_cachebook_destroy": (c_int32, [PP]),
            "llm_cachebook_open": (c_int32, [PP, I32P]), "llm_cachebook_close": (c_int32, [PP, c_int32]),
            "llm_cachebook_reserve": (c_int32, [PP, c_int32, I32P, I32P]), "llm_cachebook_commit": (c_int32, [PP, c_int32, c_int32]),
            "llm_cachebook_page_table": (c_int32, [PP, c_int32, c_int32, I32P, c_int32, I32P]),
            "llm_cachebook_check": (c_int32, [PP]), "llm_cachebook_info": (c_int32, [PP, PP]),
            "llm_debug_pool_script": (c_int32, [PP, PP]),
            "llm_part_build": (c_int32, [PP, c_char_p, PP, c_char_p, c_int64]), "llm_part_destroy": (c_int32, [PP]),
            "llm_part_describe": (c_int32, [PP, PP]), "llm_part_forward": (c_int32, [PP, PP, PP]),
            "llm_part_load": (c_int32, [PP, c_int32, POINTER(c_char_p), POINTER(c_char_p), POINTER(I64P), I32P, POINTER(c_void_p)]),
            "llm_register_part": (c_int32, [c_char_p, c_char_p, c_void_p, c_int32]),
            "llm_register_architecture": (c_int32, [c_char_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int32]),
        }
        for name, (res, args) in sigs.items():
            f = getattr(L, name)
            f.restype, f.argtypes = res, args
        L.llm_init.restype = None
        L.llm_init()
        _lib = L
    return _lib


def raise_last(status: int) -> None:
    L = lib()
    msg = (L.llm_get_last_error_message() or b"").decode("utf-8", "replace")
    kind = L.llm_get_last_error_kind()
    cls = _KINDS.get(kind, errors.LlmError)
    if cls is errors.WeightsError:
        d = json.loads((L.llm_get_last_error_details() or b"{}").decode("utf-8", "replace"))
        wrong = [(n, tuple(a), tuple(b)) for n, a, b in d.get("wrong_shape", [])]
        raise errors.WeightsError(msg, d.get("missing", []), d.get("unexpected", []), wrong)
    raise cls(msg)


def check(status: int) -> None:
    if status != 0:
        raise_last(status)


class Json(c_void_p):
    """An llm_json_t that frees itself; ``Json(obj)`` holds obj, ``.get()`` reads it back.  It is
    its own handle, so ``byref`` of it (``.ref``) keeps it alive for the length of a call."""

    def __init__(self, obj: Any = None):
        super().__init__()
        check(lib().llm_json_init(ctypes.byref(self)))
        if obj is not None:
            self.set(obj)

    def set(self, obj: Any) -> None:
        check(lib().llm_json_parse(ctypes.byref(self), json.dumps(obj).encode("utf-8")))

    def get(self) -> Any:
        L = lib()
        n = L.llm_json_dump_size(ctypes.byref(self))
        buf = ctypes.create_string_buffer(int(n))
        check(L.llm_json_dump(ctypes.byref(self), buf, n))
        return json.loads(buf.value.decode("utf-8"))

    @property
    def ref(self):
        return ctypes.byref(self)

    def __del__(self):
        try:
            lib().llm_json_destroy(ctypes.byref(self))
        except Exception:
            pass


_NP_CODES = {"float32": "F32", "float16": "F16", "float64": "F64", "int64": "I64", "int32": "I32", "int16": "I16",
             "int8": "I8", "uint8": "U8", "bool": "BOOL", "bfloat16": "BF16"}


def host_tensors(tensors) -> tuple:
    """(n, names, dtypes, shapes, ndims, pointers, keep) for a dict name -> numpy array or CPU torch
    tensor, as the C interface takes tensors in host memory.  ``keep`` must outlive the call."""
    names, dtypes, shapes, ndims, ptrs, keep = [], [], [], [], [], []
    for name, t in tensors.items():
        if hasattr(t, "detach"):                       # a torch tensor
            t = t.detach().cpu().contiguous()
            code = _NP_CODES.get(str(t.dtype).replace("torch.", ""))
            ptr, shape = t.data_ptr(), list(t.shape)
        else:
            import numpy as np
            t = np.ascontiguousarray(t)
            code = _NP_CODES.get(str(t.dtype))
            ptr, shape = t.ctypes.data, list(t.shape)
        if code is None:
            raise errors.InvalidArgError(f"tensor '{name}': element type {t.dtype} cannot be handed over")
        arr = (c_int64 * max(1, len(shape)))(*shape)
        keep.extend([t, arr])
        names.append(name.encode())
        dtypes.append(code.encode())
        shapes.append(ctypes.cast(arr, POINTER(c_int64)))
        ndims.append(len(shape))
        ptrs.append(ptr)
    n = len(names)
    return (n, (c_char_p * max(1, n))(*names), (c_char_p * max(1, n))(*dtypes), (POINTER(c_int64) * max(1, n))(*shapes),
            (c_int32 * max(1, n))(*ndims), (c_void_p * max(1, n))(*ptrs), keep)


def int32_array(values: Sequence[int]):
    return (c_int32 * max(1, len(values)))(*values)


def use_families(families: Sequence[str]) -> None:
    """Builds the kernel families and tells the host library where they lie."""
    families = [f for f in families if f not in _registered]
    if not families:
        return
    paths = build.ensure_built(families)
    L = lib()
    for fam, path in zip(families, paths):
        check(L.llm_set_kernel_library(fam.encode(), path.encode()))
        _registered.add(fam)


def describe_model(config_json: dict, dtype: str = "bfloat16") -> dict:
    out = Json()
    check(lib().llm_describe_model(Json(config_json).ref, dtype.encode(), out.ref))
    return out.get()


def kernel_families_for(folder: str, dtype: str = "bfloat16") -> List[str]:
    import os
    with open(os.path.join(folder, "config.json")) as f:
        return describe_model(json.load(f), dtype)["kernel_families"]
