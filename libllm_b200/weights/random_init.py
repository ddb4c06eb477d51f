"""Random weights from a configuration and a seed, and a model folder made of them.

Matrices are N(0, 0.02), norm weights 1 + U(-0.1, 0.1).  Each tensor draws from its
own generator seeded with (seed, CRC-32 of its name), so a tensor's values depend
neither on the order of the list nor on which other tensors the model has.  The
reference has no random model (only random tensors for operator tests,
src/flint/cuda/test.cc)."""
from __future__ import annotations

import json
import os
import zlib
from typing import Dict, Iterable

import torch

from .safetensors_io import write_safetensors
from .state_map import SINGLE_NAME, TensorNeed


def _generator(seed: int, name: str, device) -> torch.Generator:
    g = torch.Generator(device=device)
    g.manual_seed((int(seed) * 1000003 + zlib.crc32(name.encode("utf-8"))) % (2 ** 63 - 1))
    return g


def random_tensor(need: TensorNeed, seed: int, dtype: torch.dtype, device="cpu",
                  std: float = 0.02) -> torch.Tensor:
    g = _generator(seed, need.name, device)
    if need.role == "table":
        raise ValueError(f"{need.name}: integer tables have no random form")
    if need.role == "vector" and need.name.endswith("bias"):
        t = torch.empty(need.shape, dtype=torch.float32, device=device).normal_(0.0, std, generator=g)
    elif need.role == "vector":
        t = torch.empty(need.shape, dtype=torch.float32, device=device).uniform_(-0.1, 0.1, generator=g) + 1.0
    else:
        t = torch.empty(need.shape, dtype=torch.float32, device=device).normal_(0.0, std, generator=g)
    return t.to(dtype)


def random_state(needs: Iterable[TensorNeed], seed: int, dtype: torch.dtype = torch.bfloat16,
                 device="cpu") -> Dict[str, torch.Tensor]:
    """A tensor for every non-optional need, in the storage type ``dtype``."""
    return {n.name: random_tensor(n, seed, dtype, device) for n in needs if not n.optional}


def write_model_folder(folder: str, config_json: dict, tensors: Dict[str, torch.Tensor]) -> None:
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(config_json, f, indent=1)
    write_safetensors(os.path.join(folder, SINGLE_NAME), tensors, {"format": "pt"})
