"""The cache's bookkeeping as Python sees it, for inspection and tests: the host library's own
classes (cache/pages.cc, cache/kv_cache.cc) without device storage."""
from __future__ import annotations

import ctypes
from ctypes import c_int32, c_void_p
from typing import Any, Dict, List, Optional, Sequence

import numpy as np

from .. import _lib


class CacheBook:
    """The books of a cache: ``runs[i]`` is what schedule entry i wants cached (None: nothing of
    its own; else {"kind", "n_kv_heads", "k_dim", "v_dim", "window"}), ``states[i]`` its fixed-size
    state tensors [{"name", "shape"}]."""

    def __init__(self, runs: Sequence[Optional[Dict[str, Any]]], states: Sequence[Sequence[Dict[str, Any]]] = (),
                 capacity_tokens: int = 64, page_size: int = 64, max_slots: Optional[int] = None):
        self._h = c_void_p()
        spec = dict(runs=list(runs), states=[list(s) for s in states], capacity_tokens=capacity_tokens,
                    page_size=page_size, max_slots=max_slots or 0)
        _lib.check(_lib.lib().llm_cachebook_init(ctypes.byref(self._h), _lib.Json(spec).ref))

    def open(self) -> int:
        s = c_int32()
        _lib.check(_lib.lib().llm_cachebook_open(ctypes.byref(self._h), ctypes.byref(s)))
        return s.value

    def close(self, slot: int) -> None:
        _lib.check(_lib.lib().llm_cachebook_close(ctypes.byref(self._h), int(slot)))

    def reserve(self, growth: Dict[int, int]) -> None:
        slots, lens = list(growth.keys()), list(growth.values())
        _lib.check(_lib.lib().llm_cachebook_reserve(ctypes.byref(self._h), len(slots), _lib.int32_array(slots),
                                                    _lib.int32_array(lens)))

    def commit(self, slot: int, new_len: int) -> None:
        _lib.check(_lib.lib().llm_cachebook_commit(ctypes.byref(self._h), int(slot), int(new_len)))

    def page_table(self, group: int, slots: Sequence[int], width: int) -> np.ndarray:
        out = np.zeros((len(slots), width), dtype=np.int32)
        _lib.check(_lib.lib().llm_cachebook_page_table(ctypes.byref(self._h), int(group), len(slots), _lib.int32_array(list(slots)),
                                                       int(width), out.ctypes.data_as(ctypes.POINTER(c_int32))))
        return out

    def check(self) -> None:
        _lib.check(_lib.lib().llm_cachebook_check(ctypes.byref(self._h)))

    def info(self) -> Dict[str, Any]:
        out = _lib.Json()
        _lib.check(_lib.lib().llm_cachebook_info(ctypes.byref(self._h), out.ref))
        return out.get()

    def __del__(self):
        try:
            if self._h:
                _lib.lib().llm_cachebook_destroy(ctypes.byref(self._h))
        except Exception:
            pass


def pool_script(kind: str, n: int, ops: Sequence[Dict[str, Any]]) -> List[Dict[str, Any]]:
    """Runs operations on a page pool ("pages") or a slot table ("slots") of the host library and
    returns, per operation, {"result", "error", "available", "in_use"}.  Operations: {"op": "take",
    "n": k}, {"op": "give_back", "pages": [...]} or {"op": "give_back", "slot": s}, {"op": "check"},
    {"op": "held"}."""
    out = _lib.Json()
    _lib.check(_lib.lib().llm_debug_pool_script(_lib.Json(dict(kind=kind, n=n, ops=list(ops))).ref, out.ref))
    return out.get()


__all__ = ["CacheBook", "pool_script"]
