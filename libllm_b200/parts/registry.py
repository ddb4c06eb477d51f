"""Registry of part classes: (category, kind) -> class.

Categories are "norm", "position", "mixer", "feed_forward" and "block".  A new part
registers itself with ``register_part`` and is then chosen by any spec that carries its
kind; no file of the library has to change for that."""
from __future__ import annotations

from typing import Dict, Tuple

from ..errors import ConfigError

CATEGORIES = ("norm", "position", "mixer", "feed_forward", "block")
_PARTS: Dict[Tuple[str, str], type] = {}


def register_part(category: str, kind: str, cls: type, replace: bool = False) -> type:
    if category not in CATEGORIES:
        raise ConfigError(f"unknown part category '{category}' (one of {', '.join(CATEGORIES)})")
    if (category, kind) in _PARTS and not replace:
        raise ConfigError(f"{category} '{kind}' is registered already")
    _PARTS[(category, kind)] = cls
    return cls


def part(category: str, kind: str):
    """Class decorator form of ``register_part``."""
    def deco(cls):
        return register_part(category, kind, cls)
    return deco


def part_class(category: str, kind: str) -> type:
    try:
        return _PARTS[(category, kind)]
    except KeyError:
        known = sorted(k for c, k in _PARTS if c == category)
        raise ConfigError(f"no {category} of kind '{kind}' is registered (known: {', '.join(known)})") from None


def build_part(category: str, spec, env):
    return part_class(category, spec.kind)(spec, env)
