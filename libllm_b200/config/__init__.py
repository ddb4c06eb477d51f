"""Configuration and the registry of architectures, as Python sees them.  Parsing, checking and
the registry itself are the host library's (config/config.cc, config/llama.cc); a configuration is
a dict in the architecture's normal form (config.json's own keys, every one present)."""
from __future__ import annotations

import ctypes
import json
from typing import Any, Callable, Dict, List, Optional

from .. import _lib
from ..errors import ConfigError

_kept = []          # callbacks handed to the host library must outlive it


def known_architectures() -> List[str]:
    out = _lib.Json()
    _lib.check(_lib.lib().llm_known_architectures(out.ref))
    return out.get()


def load_config(folder: str) -> Dict[str, Any]:
    """config.json of ``folder``, checked and in normal form."""
    out = _lib.Json()
    _lib.check(_lib.lib().llm_load_config(folder.encode(), out.ref))
    return out.get()


def parse_config(config_json: Dict[str, Any]) -> Dict[str, Any]:
    """The same for a config.json already read; ``model_type`` picks the architecture."""
    out = _lib.Json()
    _lib.check(_lib.lib().llm_parse_config(_lib.Json(config_json).ref, out.ref))
    return out.get()


def parse_llama_config(config_json: Dict[str, Any]) -> Dict[str, Any]:
    return parse_config(dict(config_json, model_type=config_json.get("model_type", "llama")))


def describe_model(config_json: Dict[str, Any], dtype: str = "bfloat16") -> Dict[str, Any]:
    """{"spec": the model as data, "tensor_needs", "kernel_families", "capturable"}."""
    return _lib.describe_model(config_json, dtype)


def register_architecture(name: str, parse: Optional[Callable[[dict], dict]], describe: Optional[Callable[[dict], dict]],
                          replace: bool = False) -> None:
    """An architecture defined in Python: ``parse(config.json dict) -> normal form`` and
    ``describe(normal form) -> model description`` (the keys of parts/spec.h: ModelSpec)."""
    L = _lib.lib()
    if parse is None or describe is None:
        _lib.check(L.llm_register_architecture(name.encode(), None, None, None, None, int(replace)))
        return
    state = {"error": b"", "text": b""}
    FN = ctypes.CFUNCTYPE(ctypes.c_void_p, ctypes.c_char_p, ctypes.c_void_p)
    ERR = ctypes.CFUNCTYPE(ctypes.c_void_p, ctypes.c_void_p)

    def wrap(fn):
        def call(text, _user):
            try:
                state["text"] = ctypes.create_string_buffer(json.dumps(fn(json.loads(text.decode()))).encode())
                return ctypes.addressof(state["text"])
            except Exception as e:              # reported through last_error
                state["error"] = ctypes.create_string_buffer(f"{type(e).__name__}: {e}".encode())
                return None
        return FN(call)

    def last_error(_user):
        return ctypes.addressof(state["error"]) if state["error"] else None

    c_parse, c_describe, c_err = wrap(parse), wrap(describe), ERR(last_error)
    _kept.extend([c_parse, c_describe, c_err, state])
    _lib.check(L.llm_register_architecture(name.encode(), ctypes.cast(c_parse, ctypes.c_void_p),
                                           ctypes.cast(c_describe, ctypes.c_void_p), ctypes.cast(c_err, ctypes.c_void_p),
                                           None, int(replace)))


__all__ = ["known_architectures", "load_config", "parse_config", "parse_llama_config", "describe_model",
           "register_architecture", "ConfigError"]
