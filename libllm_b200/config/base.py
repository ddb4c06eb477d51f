"""Typed configuration and the one registry from an architecture's name to its model.

The reference keeps one typed struct per architecture, filled key by key from the
model's own configuration section, and picks the model class by the ``type`` string
(src/libllm/llama.cc:53-75, src/libllm/model_for_generation.cc:33-52).  Here the keys
are those of the checkpoint's config.json, the struct is a frozen dataclass, and the
``if type == ...`` chain is a table that other architectures add themselves to."""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Any, Callable, Dict, Mapping, Tuple

from ..errors import ConfigError

_MISSING = object()


class ConfigReader:
    """Reads keys of one config.json with type checks and remembers which were read."""

    def __init__(self, data: Mapping[str, Any], where: str = "config.json"):
        self.data = data
        self.where = where

    def _get(self, key, default):
        if key in self.data and self.data[key] is not None:
            return self.data[key]
        if default is _MISSING:
            raise ConfigError(f"{self.where}: required key '{key}' is missing")
        return default

    def integer(self, key: str, default=_MISSING, minimum: int = 1) -> int:
        v = self._get(key, default)
        if v is None:
            return v
        if isinstance(v, bool) or not isinstance(v, int):
            raise ConfigError(f"{self.where}: '{key}' must be an integer, found {v!r}")
        if v < minimum:
            raise ConfigError(f"{self.where}: '{key}' must be at least {minimum}, found {v}")
        return v

    def number(self, key: str, default=_MISSING, positive: bool = True) -> float:
        v = self._get(key, default)
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            raise ConfigError(f"{self.where}: '{key}' must be a number, found {v!r}")
        if positive and not v > 0:
            raise ConfigError(f"{self.where}: '{key}' must be positive, found {v}")
        return float(v)

    def boolean(self, key: str, default=_MISSING) -> bool:
        v = self._get(key, default)
        if not isinstance(v, bool):
            raise ConfigError(f"{self.where}: '{key}' must be true or false, found {v!r}")
        return v

    def string(self, key: str, default=_MISSING) -> str:
        v = self._get(key, default)
        if not isinstance(v, str):
            raise ConfigError(f"{self.where}: '{key}' must be a string, found {v!r}")
        return v

    def raw(self, key: str, default=None):
        return self.data.get(key, default)


@dataclass(frozen=True)
class ModelConfig:
    """What every architecture's configuration has in common."""
    model_type: str

    def to_json_dict(self) -> Dict[str, Any]:
        raise NotImplementedError


@dataclass(frozen=True)
class Architecture:
    """One entry of the registry.

    ``parse`` turns the config.json dict into the architecture's typed configuration;
    ``describe`` turns that configuration into a ``ModelSpec`` (libllm_b200/parts/spec.py):
    the layers, the parts each is made of, the order they run in and the names of
    their tensors.  Nothing else in the library knows the architecture's name."""
    name: str
    parse: Callable[[Mapping[str, Any]], ModelConfig]
    describe: Callable[[ModelConfig], Any]


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(name: str, parse, describe, replace: bool = False) -> None:
    if name in _ARCHITECTURES and not replace:
        raise ConfigError(f"architecture '{name}' is registered already")
    _ARCHITECTURES[name] = Architecture(name, parse, describe)


def known_architectures() -> Tuple[str, ...]:
    return tuple(sorted(_ARCHITECTURES))


def architecture_for(model_type: str) -> Architecture:
    """The registry lookup; an unknown name is an error that lists the known ones
    (the reference: "unexpected model type", src/libllm/model_for_generation.cc:47-49)."""
    try:
        return _ARCHITECTURES[model_type]
    except KeyError:
        raise ConfigError(
            f"unexpected model type '{model_type}'; registered: {', '.join(known_architectures())}"
        ) from None


def read_config_json(folder: str) -> Dict[str, Any]:
    path = os.path.join(folder, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"{path}: no such file")
    try:
        with open(path) as f:
            data = json.load(f)
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path}: not valid JSON ({e})") from None
    if not isinstance(data, dict):
        raise ConfigError(f"{path}: the top level must be an object")
    return data


def load_config(folder: str) -> ModelConfig:
    """config.json of ``folder`` as the typed configuration of its architecture."""
    data = read_config_json(folder)
    if "model_type" not in data:
        raise ConfigError(f"{folder}/config.json: required key 'model_type' is missing")
    return architecture_for(data["model_type"]).parse(data)
