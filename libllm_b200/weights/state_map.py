"""Weights by tensor name.

``StateMap`` is the table of a model folder's tensors (one ``model.safetensors`` or the
shards an index file names).  A model states what it needs as a list of
``TensorNeed`` and gets back either every tensor or ONE error that lists all that is
missing, all that is unexpected and every wrong shape.  The reference fails at the
first tensor it cannot find or whose shape differs (src/libllm/var_builder.cc:97-140);
the messages here keep its wording per tensor.

Precision: a tensor is handed over as it is stored, except that 16-bit floats become
bfloat16 (float32 when the engine runs in float32), integer tables become int32, and a
tensor stored in 32-bit stays in 32-bit unless the need says that it feeds a matrix
product, which takes its operands in the engine's type."""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

import torch

from ..errors import WeightsError
from .safetensors_io import SafetensorsFile

INDEX_NAME = "model.safetensors.index.json"
SINGLE_NAME = "model.safetensors"


@dataclass(frozen=True)
class TensorNeed:
    """One tensor a part asks for: checkpoint name, shape, and how it is used.

    ``role`` is "matrix" (operand of a product: converted to the engine's type),
    "vector" (norm weights, biases: kept in 32-bit if stored so, else widened to the
    engine's accumulate type by the part) or "table" (integers)."""
    name: str
    shape: Tuple[int, ...]
    role: str = "matrix"
    optional: bool = False


class StateMap:
    """Tensor name -> tensor over the files of a model folder, or over a plain dict."""

    def __init__(self, files: Sequence[SafetensorsFile] = (), tensors: Dict[str, torch.Tensor] = None,
                 where: str = "<memory>"):
        self.where = where
        self._files = list(files)
        self._mem = dict(tensors or {})
        self._index: Dict[str, SafetensorsFile] = {}
        for f in self._files:
            for n in f.names():
                if n in self._index:
                    raise WeightsError(f"{where}: tensor '{n}' is stored twice "
                                       f"({self._index[n].path} and {f.path})")
                self._index[n] = f

    @classmethod
    def from_folder(cls, folder: str) -> "StateMap":
        idx = os.path.join(folder, INDEX_NAME)
        single = os.path.join(folder, SINGLE_NAME)
        if os.path.isfile(idx):
            with open(idx) as f:
                wm = json.load(f).get("weight_map", {})
            names = sorted(set(wm.values()))
            missing = [n for n in names if not os.path.isfile(os.path.join(folder, n))]
            if missing:
                raise WeightsError(f"{folder}: shard files named by {INDEX_NAME} are missing: "
                                   + ", ".join(missing))
            files = [SafetensorsFile(os.path.join(folder, n)) for n in names]
        elif os.path.isfile(single):
            files = [SafetensorsFile(single)]
        else:
            raise WeightsError(f"{folder}: neither {SINGLE_NAME} nor {INDEX_NAME} found")
        return cls(files, where=folder)

    @classmethod
    def from_tensors(cls, tensors: Dict[str, torch.Tensor]) -> "StateMap":
        return cls(tensors=tensors)

    def names(self) -> List[str]:
        return list(self._index) + list(self._mem)

    def has(self, name: str) -> bool:
        return name in self._index or name in self._mem

    def shape(self, name: str) -> Tuple[int, ...]:
        if name in self._mem:
            return tuple(self._mem[name].shape)
        return self._index[name].shape(name)

    def stored_dtype(self, name: str) -> torch.dtype:
        if name in self._mem:
            return self._mem[name].dtype
        return self._index[name].dtype(name)

    def raw(self, name: str) -> torch.Tensor:
        if name in self._mem:
            return self._mem[name]
        return self._index[name].tensor(name)

    def check(self, needs: Iterable[TensorNeed], allow_unexpected: Iterable[str] = ()) -> None:
        """Raises one WeightsError naming every missing, unexpected and misshapen tensor."""
        needs = list(needs)
        wanted = {n.name for n in needs}
        missing = [n.name for n in needs if not n.optional and not self.has(n.name)]
        allowed = set(allow_unexpected)
        unexpected = sorted(n for n in self.names() if n not in wanted and n not in allowed)
        wrong = []
        for n in needs:
            if self.has(n.name) and tuple(self.shape(n.name)) != tuple(n.shape):
                wrong.append((n.name, tuple(n.shape), tuple(self.shape(n.name))))
        if not (missing or unexpected or wrong):
            return
        lines = [f"{self.where}: the weights do not fit the model "
                 f"({len(missing)} missing, {len(unexpected)} unexpected, {len(wrong)} with a wrong shape)"]
        for m in missing:
            lines.append(f'  missing: tensor "{m}" not found in model.')
        for u in unexpected:
            lines.append(f'  unexpected: tensor "{u}" is in the files but no part of the model asks for it.')
        for name, want, got in wrong:
            lines.append(f"  wrong shape: {name}: invalid shape: {want} expected, but {got} found.")
        raise WeightsError("\n".join(lines), missing, unexpected, wrong)

    def fetch(self, need: TensorNeed, engine_dtype: torch.dtype, device) -> Optional[torch.Tensor]:
        """The tensor of ``need`` on ``device`` in the precision its role calls for."""
        if not self.has(need.name):
            if need.optional:
                return None
            raise WeightsError(f'tensor "{need.name}" not found in model.', [need.name])
        t = self.raw(need.name)
        if tuple(t.shape) != tuple(need.shape):
            raise WeightsError(f"{need.name}: invalid shape: {tuple(need.shape)} expected, but "
                               f"{tuple(t.shape)} found.", wrong_shape=[(need.name, need.shape, tuple(t.shape))])
        if need.role == "table":
            if t.dtype.is_floating_point:
                raise WeightsError(f"{need.name}: an integer table is stored as {t.dtype}")
            return t.to(device=device, dtype=torch.int32)
        if not t.dtype.is_floating_point:
            raise WeightsError(f"{need.name}: stored as {t.dtype}, a floating-point tensor is needed")
        if need.role == "matrix":
            target = engine_dtype
        elif t.dtype in (torch.float32, torch.float64):
            target = torch.float32
        else:
            target = engine_dtype
        return t.to(device=device, dtype=target).contiguous()

    def close(self) -> None:
        for f in self._files:
            f.close()
        self._files = []
        self._index = {}
