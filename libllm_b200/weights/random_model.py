"""The random-weights mode: a model folder (config.json, model.safetensors) from a
configuration and a seed."""
from __future__ import annotations

from typing import Dict, Mapping

import torch

from ..config import architecture_for
from .random_init import random_state, write_model_folder


def tensor_needs_of(config_json: Mapping):
    """The tensors the architecture named by ``config_json`` asks for, and its typed config."""
    from ..engine.model import Model
    arch = architecture_for(config_json["model_type"])
    config = arch.parse(config_json)
    model = Model(config, arch.describe(config), torch.bfloat16, "cpu")
    return config, model.tensor_needs()


def random_tensors(config_json: Mapping, seed: int, dtype: torch.dtype = torch.bfloat16,
                   device="cpu") -> Dict[str, torch.Tensor]:
    _, needs = tensor_needs_of(config_json)
    return random_state(needs, seed, dtype, device)


def create_random_model(folder: str, config_json: Mapping, seed: int,
                        dtype: torch.dtype = torch.bfloat16, device="cpu") -> None:
    """Writes ``folder`` with config.json as given and random tensors under the names and
    shapes the architecture asks for (matrices N(0, 0.02), norm weights 1 + U(-0.1, 0.1))."""
    tensors = random_tensors(config_json, seed, dtype, device)
    write_model_folder(folder, dict(config_json), tensors)
