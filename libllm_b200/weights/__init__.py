"""Weights, as Python sees them: the random-weights mode that writes a model folder, and the
check of a folder's tensors against a list of needs.  Reading safetensors, the one error that
lists everything that does not fit, and the conversion to the device are the host library's
(weights/safetensors.cc, weights/state_map.cc)."""
from __future__ import annotations

from typing import Any, Dict, List, Optional, Sequence

from .. import _lib


def create_random_model(folder: str, config_json: Dict[str, Any], seed: int, dtype: str = "bfloat16") -> None:
    """Writes ``folder`` with config.json as given and model.safetensors with random tensors under
    the names and shapes the architecture asks for (matrices N(0, 0.02), norm weights
    1 + U(-0.1, 0.1)), each drawn from (seed, its name)."""
    _lib.check(_lib.lib().llm_create_random_model(folder.encode(), _lib.Json(dict(config_json)).ref, int(seed),
                                                  str(dtype).replace("torch.", "").encode()))


def tensor_needs_of(config_json: Dict[str, Any], dtype: str = "bfloat16") -> List[Dict[str, Any]]:
    """The tensors the architecture named by ``config_json`` asks for: name, shape, role, optional."""
    return _lib.describe_model(dict(config_json), dtype)["tensor_needs"]


def check_weights(folder: str, needs: Sequence[Dict[str, Any]], ignore: Sequence[str] = (), strict: bool = True) -> Dict[str, Any]:
    """Raises one WeightsError naming every missing, unexpected and misshapen tensor of the folder;
    otherwise returns {"missing", "unexpected", "ignored", "names"}."""
    out = _lib.Json()
    _lib.check(_lib.lib().llm_check_weights(folder.encode(), _lib.Json(list(needs)).ref, _lib.Json(list(ignore)).ref,
                                            int(strict), out.ref))
    return out.get()


def read_safetensors_header(path: str) -> Dict[str, Any]:
    """name -> {"dtype", "shape", "nbytes"} of one file; raises WeightsError for a broken file."""
    out = _lib.Json()
    _lib.check(_lib.lib().llm_read_safetensors_header(path.encode(), out.ref))
    return out.get()


__all__ = ["create_random_model", "tensor_needs_of", "check_weights", "read_safetensors_header"]
