"""Descriptions of a model as data: which parts each layer is made of, with every size
and constant as a field, the order in which layers run, and the names of their tensors.

An architecture (libllm_b200/models/) turns its configuration into one ``ModelSpec``;
the generic model (libllm_b200/engine/model.py) builds the parts each spec names through
the part registry (libllm_b200/parts/registry.py).  A spec knows nothing about the model
it is used in.  The reference builds its one architecture in code
(src/libllm/llama.cc:111-141, 231-249, 273-292); the fields here are the arguments of
those build functions."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Optional, Tuple


@dataclass(frozen=True)
class PartSpec:
    """Base of all part descriptions; ``kind`` selects the class in the registry."""
    kind: str


@dataclass(frozen=True)
class RMSNormSpec(PartSpec):
    size: int = 0
    eps: float = 0.0
    weight: str = ""            # tensor name


@dataclass(frozen=True)
class RopeSpec(PartSpec):
    """Rotary position encoding over the first ``rotary_dim`` channels of a head."""
    head_dim: int = 0
    rotary_dim: int = 0
    theta: float = 10000.0
    scaling: Any = None          # config.llama.RopeScaling or None


@dataclass(frozen=True)
class AttentionSpec(PartSpec):
    hidden: int = 0
    n_heads: int = 0
    n_kv_heads: int = 0
    head_dim: int = 0
    position: Optional[PartSpec] = None
    window: Optional[int] = None         # None: every earlier key is seen
    scale: Optional[float] = None        # None: 1/sqrt(head_dim)
    bias: bool = False                   # bias on q, k and v
    q: str = ""
    k: str = ""
    v: str = ""
    o: str = ""


@dataclass(frozen=True)
class SwiGLUSpec(PartSpec):
    hidden: int = 0
    intermediate: int = 0
    gate: str = ""
    up: str = ""
    down: str = ""


@dataclass(frozen=True)
class BlockSpec(PartSpec):
    """One layer: how a mixer and a feed-forward, each behind its norm, join the
    residual stream.  kind "prenorm": x + mixer(norm(x)), then h + ff(norm(h))."""
    mixer_norm: Optional[PartSpec] = None
    mixer: Optional[PartSpec] = None
    ff_norm: Optional[PartSpec] = None
    ff: Optional[PartSpec] = None


@dataclass(frozen=True)
class ScheduleEntry:
    """One run of a layer.  ``layer`` indexes ``ModelSpec.layers``; the same layer may
    be named by several entries (its weights are then used twice, each run with a cache
    of its own).  ``cache_from`` names an earlier entry whose cache this run reads
    instead of keeping one: it then appends nothing."""
    layer: int
    cache_from: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    vocab_size: int
    hidden: int
    embedding: str                               # tensor name of the token table
    layers: Tuple[BlockSpec, ...]
    schedule: Tuple[ScheduleEntry, ...]
    final_norm: PartSpec
    head: Optional[str]                          # output matrix; None: the token table
    max_positions: int
    stop_tokens: Tuple[int, ...] = ()
    name: str = ""
