"""Parts of one's own, defined in Python, for the host library's engine.

The parts the library brings (RMSNorm, rotary position encoding, attention over the paged cache,
SwiGLU, the pre-norm block) are C++ (parts/builtin.cc).  A mixer, a feed-forward or a position
encoding written in Python registers through the C interface of ``include/llm_plugin.h``: a
class with the methods below, ``register_part(category, kind, cls)``, and from then on any model
description that names ``kind`` builds it and the engine steps it like its own parts.  Such a
part computes on the device with whatever it likes (the tests use torch on the step's stream);
it gets device memory as ``DeviceTensor`` views.

    class MyMixer:
        capturable = False                   # True: launches on step.stream only, allocates nothing
        def __init__(self, spec: dict, env: dict): ...      # env: dtype, max_positions, page_size
        def tensor_needs(self) -> list: ...                 # [{"name", "shape", "role", "optional"}]
        def load_tensor(self, name, tensor): ...            # once per tensor, on the device
        def needs(self) -> dict: ...                        # {"cache": None | {...}, "state": [{"name", "shape", "dtype"}]}
        def forward(self, step, x, cache, state, out): ...  # writes out [T, hidden] float32

A feed-forward has ``forward(self, step, x, out)`` and no ``needs``; a position encoding has
``table(self) -> (device pointer, rows, rotary_dim)`` of a rotation that pairs channel i with
i + rotary_dim/2 (cosines, then sines, float32)."""
from __future__ import annotations

import contextlib
import ctypes
import json
from ctypes import (CFUNCTYPE, POINTER, Structure, c_char_p, c_float, c_int32, c_int64, c_void_p)
from typing import Any, Dict, List, Optional, Tuple

from .. import _lib

DTYPE_NAMES = {0: "float32", 1: "bfloat16", 2: "int32"}
_ITEMSIZE = {"float32": 4, "bfloat16": 2, "int32": 4}
_TYPESTR = {"float32": "<f4", "bfloat16": "<i2", "int32": "<i4"}


class DeviceTensor:
    """A view of device memory: pointer, element type, shape and row strides (in elements)."""

    def __init__(self, ptr: int, dtype: str, shape, strides=None):
        self.ptr, self.dtype, self.shape = int(ptr or 0), dtype, tuple(int(s) for s in shape)
        if strides is None:
            strides, acc = [], 1
            for s in reversed(self.shape):
                strides.insert(0, acc)
                acc *= s
        self.strides = tuple(int(s) for s in strides)

    @property
    def __cuda_array_interface__(self):
        item = _ITEMSIZE[self.dtype]
        return dict(shape=self.shape, typestr=_TYPESTR[self.dtype], data=(self.ptr, False), version=3,
                    strides=tuple(s * item for s in self.strides))

    def torch(self):
        """The same memory as a torch tensor (nothing is copied)."""
        import torch
        if 0 in self.shape or self.ptr == 0:
            return torch.empty(self.shape, dtype=getattr(torch, self.dtype), device="cuda")
        t = torch.as_tensor(self, device="cuda")
        return t.view(torch.bfloat16) if self.dtype == "bfloat16" else t


class _Act(Structure):
    _fields_ = [("data", c_void_p), ("dtype", c_int32), ("rows", c_int64), ("cols", c_int64), ("ld", c_int64),
                ("parts", c_int32), ("part_stride", c_int64)]

    def view(self) -> DeviceTensor:
        name = DTYPE_NAMES[self.dtype]
        if self.parts > 1:
            return DeviceTensor(self.data, name, (self.parts, self.rows, self.cols), (self.part_stride, self.ld, 1))
        return DeviceTensor(self.data, name, (self.rows, self.cols), (self.ld, 1))


class _Step(Structure):
    _fields_ = [("dtype", c_int32), ("stream", c_void_p), ("n_tokens", c_int32), ("n_seqs", c_int32), ("n_want", c_int32),
                ("tokens", c_void_p), ("tok_seq", c_void_p), ("tok_pos", c_void_p), ("seq_start", c_void_p),
                ("seq_past", c_void_p), ("seq_slot", c_void_p), ("want_rows", c_void_p),
                ("q_lens", POINTER(c_int32)), ("past_lens", POINTER(c_int32)), ("slots", POINTER(c_int32)),
                ("max_q_len", c_int32), ("max_kv_len", c_int32), ("decode_only", c_int32), ("captured", c_int32)]


class _LayerCache(Structure):
    _fields_ = [("k", c_void_p), ("v", c_void_p), ("n_pages", c_int64), ("page_table", c_void_p), ("table_width", c_int32),
                ("page_size", c_int32), ("writes", c_int32), ("group", c_int32), ("dtype", c_int32),
                ("n_kv_heads", c_int32), ("k_dim", c_int32), ("v_dim", c_int32), ("window", c_int32)]


class _StateTensor(Structure):
    _fields_ = [("name", c_char_p), ("data", c_void_p), ("ndim", c_int32), ("shape", c_int64 * 4), ("dtype", c_int32),
                ("n_slots", c_int64)]


class Step:
    """One step as a part sees it: T tokens of B sequences, each sequence's tokens contiguous.
    The ``tok_*`` and ``seq_*`` members are int32 device arrays; ``q_lens``, ``past_lens`` and
    ``slots`` are host lists (the step's own only when ``captured`` is false)."""

    def __init__(self, s: _Step):
        self.dtype = DTYPE_NAMES[s.dtype]
        self.stream = s.stream or 0
        self.n_tokens, self.n_seqs, self.n_want = s.n_tokens, s.n_seqs, s.n_want
        T, B = s.n_tokens, s.n_seqs
        self.tokens = DeviceTensor(s.tokens, "int32", (T,))
        self.tok_seq = DeviceTensor(s.tok_seq, "int32", (T,))
        self.tok_pos = DeviceTensor(s.tok_pos, "int32", (T,))
        self.seq_start = DeviceTensor(s.seq_start, "int32", (B + 1,))
        self.seq_past = DeviceTensor(s.seq_past, "int32", (B,))
        self.seq_slot = DeviceTensor(s.seq_slot, "int32", (B,))
        self.q_lens = [s.q_lens[i] for i in range(B)]
        self.past_lens = [s.past_lens[i] for i in range(B)]
        self.slots = [s.slots[i] for i in range(B)]
        self.max_q_len, self.max_kv_len = s.max_q_len, s.max_kv_len
        self.decode_only, self.captured = bool(s.decode_only), bool(s.captured)

    @contextlib.contextmanager
    def torch_stream(self):
        """Makes torch launch on the engine's stream inside the block."""
        import torch
        with torch.cuda.stream(torch.cuda.ExternalStream(self.stream)):
            yield


class Cache:
    """What a run of a layer sees of the cache: ``k`` [pages, kv_heads, page_size, k_dim], ``v``
    likewise with v_dim (None when v_dim is 0), ``page_table`` int32 [sequences, width]."""

    def __init__(self, c: _LayerCache, n_seqs: int):
        dt = DTYPE_NAMES[c.dtype]
        self.page_size, self.writes, self.group, self.window = c.page_size, bool(c.writes), c.group, c.window
        self.n_kv_heads, self.k_dim, self.v_dim = c.n_kv_heads, c.k_dim, c.v_dim
        self.k = DeviceTensor(c.k, dt, (c.n_pages, c.n_kv_heads, c.page_size, c.k_dim))
        self.v = DeviceTensor(c.v, dt, (c.n_pages, c.n_kv_heads, c.page_size, c.v_dim)) if c.v_dim else None
        self.page_table = DeviceTensor(c.page_table, "int32", (n_seqs, c.table_width))


_CREATE = CFUNCTYPE(c_void_p, c_char_p, c_char_p, c_void_p)
_DESTROY = CFUNCTYPE(None, c_void_p)
_TEXT = CFUNCTYPE(c_void_p, c_void_p)
_LOAD = CFUNCTYPE(c_int32, c_void_p, c_char_p, c_void_p, c_int32, POINTER(c_int64), c_int32)
_MIXER = CFUNCTYPE(c_int32, c_void_p, POINTER(_Step), POINTER(_Act), POINTER(_LayerCache), POINTER(_StateTensor), c_int32,
                   POINTER(_Act))
_FF = CFUNCTYPE(c_int32, c_void_p, POINTER(_Step), POINTER(_Act), POINTER(_Act))
_TABLE = CFUNCTYPE(c_void_p, c_void_p, POINTER(c_int32), POINTER(c_int32))
_ERR = CFUNCTYPE(c_void_p, c_void_p)


class _VTable(Structure):
    _fields_ = [("user", c_void_p), ("create", _CREATE), ("destroy", _DESTROY), ("tensor_needs", _TEXT), ("load_tensor", _LOAD),
                ("needs", _TEXT), ("mixer_forward", _MIXER), ("ff_forward", _FF), ("position_table", _TABLE),
                ("last_error", _ERR), ("capturable", c_int32), ("out_width", c_int64)]


_kept: List[Any] = []               # vtables and callbacks must outlive the host library's use of them
_instances: Dict[int, Any] = {}
_next_id = [1]


def register_part(category: str, kind: str, cls: type, replace: bool = False) -> type:
    """Registers a Python class as the part of ``kind`` in ``category`` ("mixer", "feed_forward" or
    "position")."""
    state = {"error": None, "texts": {}}

    def fail(e: BaseException):
        state["error"] = ctypes.create_string_buffer(f"{type(e).__name__}: {e}".encode())

    def text_of(handle: int, obj: Any) -> int:
        buf = ctypes.create_string_buffer(json.dumps(obj).encode())
        state["texts"][handle] = buf
        return ctypes.addressof(buf)

    def create(spec, env, _user):
        try:
            obj = cls(json.loads(spec.decode()), json.loads(env.decode()))
            handle = _next_id[0]
            _next_id[0] += 1
            _instances[handle] = obj
            return handle
        except BaseException as e:
            fail(e)
            return None

    def destroy(handle):
        _instances.pop(handle, None)
        state["texts"].pop(handle, None)

    def tensor_needs(handle):
        try:
            obj = _instances[handle]
            return text_of(handle, obj.tensor_needs() if hasattr(obj, "tensor_needs") else [])
        except BaseException as e:
            fail(e)
            return None

    def load_tensor(handle, name, ptr, dtype, shape, ndim):
        try:
            obj = _instances[handle]
            if hasattr(obj, "load_tensor"):
                obj.load_tensor(name.decode(), DeviceTensor(ptr, DTYPE_NAMES[dtype], [shape[i] for i in range(ndim)]))
            return 0
        except BaseException as e:
            fail(e)
            return 1

    def needs(handle):
        try:
            obj = _instances[handle]
            return text_of(handle, (obj.needs() if hasattr(obj, "needs") else None) or {})
        except BaseException as e:
            fail(e)
            return None

    def mixer_forward(handle, step, x, cache, state_p, n_state, out):
        try:
            s = Step(step.contents)
            c = Cache(cache.contents, s.n_seqs) if cache else None
            st = {}
            for i in range(n_state):
                t = state_p[i]
                st[t.name.decode()] = DeviceTensor(t.data, DTYPE_NAMES[t.dtype], (t.n_slots,) + tuple(t.shape[j] for j in range(t.ndim)))
            _instances[handle].forward(s, x.contents.view(), c, st, out.contents.view())
            return 0
        except BaseException as e:
            fail(e)
            return 1

    def ff_forward(handle, step, x, out):
        try:
            _instances[handle].forward(Step(step.contents), x.contents.view(), out.contents.view())
            return 0
        except BaseException as e:
            fail(e)
            return 1

    def position_table(handle, rows, rot):
        try:
            ptr, r, d = _instances[handle].table()
            rows[0], rot[0] = int(r), int(d)
            return int(ptr)
        except BaseException as e:
            fail(e)
            return None

    def last_error(_user):
        return ctypes.addressof(state["error"]) if state["error"] is not None else None

    vt = _VTable()
    vt.user = None
    vt.create, vt.destroy = _CREATE(create), _DESTROY(destroy)
    vt.tensor_needs, vt.load_tensor, vt.needs = _TEXT(tensor_needs), _LOAD(load_tensor), _TEXT(needs)
    if category == "mixer":
        vt.mixer_forward = _MIXER(mixer_forward)
    elif category == "feed_forward":
        vt.ff_forward = _FF(ff_forward)
    elif category == "position":
        vt.position_table = _TABLE(position_table)
    vt.last_error = _ERR(last_error)
    vt.capturable = 1 if getattr(cls, "capturable", False) else 0
    vt.out_width = int(getattr(cls, "out_width", 0) or 0)
    _kept.extend([vt, state])
    _lib.check(_lib.lib().llm_register_part(category.encode(), kind.encode(), ctypes.cast(ctypes.pointer(vt), c_void_p), int(replace)))
    return cls


class PartHandle:
    """One part of the host library alone (capi/llm_parts_api.cc): built from its description,
    given its tensors, run on device memory that the caller brings.  ``forward`` takes the call as
    a dict whose device pointers are integers (``tensor.data_ptr()``) and returns views of what
    the part produced, valid until the next call."""

    def __init__(self, category: str, spec: Dict[str, Any], dtype: str = "bfloat16", max_positions: int = 512):
        desc = _lib.Json()
        self._h = c_void_p()
        self.category = category
        # the kernels a part launches are asked for first, so that they are built and known
        probe = c_void_p()
        _lib.check(_lib.lib().llm_part_build(ctypes.byref(probe), category.encode(), _lib.Json(spec).ref, dtype.encode(),
                                             int(max_positions)))
        try:
            _lib.check(_lib.lib().llm_part_describe(ctypes.byref(probe), desc.ref))
        finally:
            _lib.lib().llm_part_destroy(ctypes.byref(probe))
        self.description = desc.get()
        _lib.use_families(self.description["kernel_families"])
        _lib.check(_lib.lib().llm_part_build(ctypes.byref(self._h), category.encode(), _lib.Json(spec).ref, dtype.encode(),
                                             int(max_positions)))

    def load(self, tensors: Dict[str, Any]) -> None:
        n, names, dtypes, shapes, ndims, ptrs, keep = _lib.host_tensors(tensors)
        _lib.check(_lib.lib().llm_part_load(ctypes.byref(self._h), n, names, dtypes, shapes, ndims, ptrs))

    def forward(self, call: Dict[str, Any]) -> Dict[str, Any]:
        out = _lib.Json()
        _lib.check(_lib.lib().llm_part_forward(ctypes.byref(self._h), _lib.Json(call).ref, out.ref))
        res = out.get()
        views: Dict[str, Any] = {}
        for key in ("out", "pending"):
            a = res.get(key)
            if a:
                shape = (a["parts"], a["rows"], a["cols"]) if a["parts"] > 1 else (a["rows"], a["cols"])
                strides = (a["part_stride"], a["ld"], 1) if a["parts"] > 1 else (a["ld"], 1)
                views[key] = DeviceTensor(a["ptr"], a["dtype"], shape, strides)
            else:
                views[key] = None
        if res.get("table"):
            t = res["table"]
            views["table"] = DeviceTensor(t["ptr"], "float32", (t["rows"], t["rotary_dim"]))
        return views

    def __del__(self):
        try:
            if self._h:
                _lib.lib().llm_part_destroy(ctypes.byref(self._h))
        except Exception:
            pass


__all__ = ["register_part", "DeviceTensor", "Step", "Cache", "PartHandle"]
