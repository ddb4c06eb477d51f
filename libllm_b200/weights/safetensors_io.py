"""Reader and writer of the safetensors container.

The file is: an 8-byte little-endian length, a JSON header of that length mapping each
tensor name to {"dtype", "shape", "data_offsets": [begin, end]} relative to the end of
the header, then the raw little-endian data.  The reference reads a container of its
own ("TDIC", src/libllm/var_builder.cc:38-95) that an offline exporter writes; reading
the checkpoint's own file takes that step's place."""
from __future__ import annotations

import json
import mmap
import os
import struct
import warnings
from typing import Dict, List, Mapping, Tuple

import numpy as np
import torch

from ..errors import WeightsError

_DTYPES = {
    "F32": (torch.float32, np.float32, 4),
    "F16": (torch.float16, np.float16, 2),
    "BF16": (torch.bfloat16, np.uint16, 2),
    "F64": (torch.float64, np.float64, 8),
    "I64": (torch.int64, np.int64, 8),
    "I32": (torch.int32, np.int32, 4),
    "I16": (torch.int16, np.int16, 2),
    "I8": (torch.int8, np.int8, 1),
    "U8": (torch.uint8, np.uint8, 1),
    "BOOL": (torch.bool, np.bool_, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


class SafetensorsFile:
    """One file, memory-mapped; ``tensor(name)`` copies nothing until it is used."""

    def __init__(self, path: str):
        self.path = path
        size = os.path.getsize(path)
        if size < 8:
            raise WeightsError(f"{path}: truncated file (no header length)")
        self._file = open(path, "rb")
        (hlen,) = struct.unpack("<Q", self._file.read(8))
        if hlen <= 0 or 8 + hlen > size:
            raise WeightsError(f"{path}: truncated file (header of {hlen} bytes, file of {size})")
        try:
            header = json.loads(self._file.read(hlen).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise WeightsError(f"{path}: invalid header ({e})") from None
        self.metadata = header.pop("__metadata__", {})
        self._base = 8 + hlen
        self.entries: Dict[str, Tuple[str, Tuple[int, ...], int, int]] = {}
        for name, e in header.items():
            dt, shape = e["dtype"], tuple(int(s) for s in e["shape"])
            b, end = (int(x) for x in e["data_offsets"])
            if dt not in _DTYPES:
                raise WeightsError(f"{path}: tensor '{name}' has unsupported dtype {dt}")
            n = 1
            for s in shape:
                n *= s
            if end - b != n * _DTYPES[dt][2] or b < 0:
                raise WeightsError(f"{path}: tensor '{name}' has {end - b} bytes, its shape needs "
                                   f"{n * _DTYPES[dt][2]}")
            if self._base + end > size:
                raise WeightsError(f"{path}: truncated file (tensor '{name}' ends at byte "
                                   f"{self._base + end}, file has {size})")
            self.entries[name] = (dt, shape, b, end)
        self._mmap = mmap.mmap(self._file.fileno(), 0, access=mmap.ACCESS_READ) if size else None

    def names(self) -> List[str]:
        return list(self.entries)

    def shape(self, name: str) -> Tuple[int, ...]:
        return self.entries[name][1]

    def dtype(self, name: str) -> torch.dtype:
        return _DTYPES[self.entries[name][0]][0]

    def tensor(self, name: str) -> torch.Tensor:
        dt, shape, b, end = self.entries[name]
        tdt, ndt, _ = _DTYPES[dt]
        arr = np.frombuffer(self._mmap, dtype=ndt, count=(end - b) // _DTYPES[dt][2],
                            offset=self._base + b)
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")     # the mapping is read-only; nothing writes to it
            t = torch.from_numpy(arr.copy() if arr.size == 0 else arr)
        if tdt == torch.bfloat16:
            t = t.view(torch.bfloat16)
        return t.reshape(shape)

    def close(self):
        if self._mmap is not None:
            self._mmap.close()
            self._mmap = None
        self._file.close()


def write_safetensors(path: str, tensors: Mapping[str, torch.Tensor],
                      metadata: Mapping[str, str] = None) -> None:
    """Writes ``tensors`` (in the mapping's order) as one safetensors file."""
    header = {}
    if metadata:
        header["__metadata__"] = dict(metadata)
    offset = 0
    order = []
    for name, t in tensors.items():
        if t.dtype not in _NAMES:
            raise WeightsError(f"tensor '{name}': dtype {t.dtype} cannot be stored")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
        order.append(name)
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name in order:
            t = tensors[name].detach().to("cpu").contiguous()
            if t.dtype == torch.bfloat16:
                t = t.view(torch.int16)
            if t.dtype == torch.bool:
                t = t.view(torch.uint8)
            f.write(t.numpy().tobytes())
