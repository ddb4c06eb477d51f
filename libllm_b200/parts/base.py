"""Interfaces of the parts a layer is put together from, and what a step hands them.

* ``Norm``          residual stream (+ pending addition) -> normalised activations
* ``PositionEncoding`` constants a mixer needs to place tokens (here: a cos/sin table)
* ``Mixer``         mixes along the sequence; may keep keys/values in the cache
                    (``cache_need``) and fixed-size state per sequence (``state_need``)
* ``FeedForward``   acts on each token alone
* ``Block``         joins a mixer and a feed-forward to the residual stream

Every part takes its sizes and constants from its spec, states the tensors it needs by
name (``tensor_needs``) and receives them through ``load``.  No part knows which model
it is in.  Activations are [tokens, width] with the step's tokens of all sequences one
after another; which token belongs to which sequence and position is in ``StepContext``.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional, Tuple

import torch

from ..weights.state_map import TensorNeed


@dataclass
class BuildEnv:
    """What a part may know about the engine it is built for."""
    dtype: torch.dtype                 # torch.float32 or torch.bfloat16
    device: torch.device
    max_positions: int                 # longest sequence the engine will hold
    page_size: int = 64


@dataclass(frozen=True)
class CacheNeed:
    """Keys and values a mixer wants kept per sequence.  ``kind`` "full" keeps every
    position, "window" only the last ``window`` (older pages are given back)."""
    kind: str
    n_kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class StateNeed:
    """One fixed-size tensor per sequence, zero when a sequence starts."""
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclass
class LayerCache:
    """The view of the cache one run of a layer gets."""
    k: torch.Tensor                    # [pages, kv_heads, page_size, d]
    v: torch.Tensor
    page_table: torch.Tensor           # int32 [sequences, pages per sequence]
    page_size: int
    writes: bool                       # False: reads another run's keys and values
    group: int = 0


@dataclass
class StepContext:
    """One step: T tokens of B sequences, each sequence's tokens contiguous."""
    dtype: torch.dtype
    device: torch.device
    n_tokens: int
    n_seqs: int
    tokens: torch.Tensor               # int32 [T]
    tok_seq: torch.Tensor              # int32 [T] index of the token's sequence in the step
    tok_pos: torch.Tensor              # int32 [T] absolute position of the token
    seq_start: torch.Tensor            # int32 [B+1] offsets of each sequence's tokens
    seq_past: torch.Tensor             # int32 [B] tokens already cached before this step
    seq_slot: torch.Tensor             # int32 [B] slot of each sequence
    want_rows: torch.Tensor            # int32 [W] token rows whose logits are asked for
    q_lens: List[int]                  # host copies
    past_lens: List[int]
    slots: List[int]
    max_q_len: int
    max_kv_len: int
    decode_only: bool                  # every sequence brings exactly one token
    kv_split_hint: int = 1             # launch-shape bucket fixed when a graph is captured
    extras: Dict[str, Any] = field(default_factory=dict)


class ResidualStream:
    """The 32-bit residual stream and an addition that has not been applied yet.  The
    addition is folded into the next norm's pass over the row."""

    def __init__(self, resid: torch.Tensor):
        self.resid = resid
        self.pending: Optional[torch.Tensor] = None


class Part:
    category = ""

    def __init__(self, spec, env: BuildEnv):
        self.spec = spec
        self.env = env

    def tensor_needs(self) -> List[TensorNeed]:
        return []

    def load(self, fetch: Callable[[TensorNeed], Optional[torch.Tensor]]) -> None:
        pass

    def kernel_families(self) -> List[str]:
        """Kernel families (libllm_b200/csrc/build.py) this part launches."""
        return []


class Norm(Part):
    category = "norm"

    def forward(self, ctx: StepContext, stream: ResidualStream,
                rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        raise NotImplementedError


class PositionEncoding(Part):
    category = "position"


class Mixer(Part):
    category = "mixer"

    def cache_need(self) -> Optional[CacheNeed]:
        return None

    def state_need(self) -> Dict[str, StateNeed]:
        return {}

    def forward(self, ctx: StepContext, x: torch.Tensor, cache: Optional[LayerCache],
                state: Optional[Dict[str, torch.Tensor]]) -> torch.Tensor:
        raise NotImplementedError


class FeedForward(Part):
    category = "feed_forward"

    def forward(self, ctx: StepContext, x: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError


class Block(Part):
    category = "block"

    def parts(self) -> List[Part]:
        raise NotImplementedError

    def mixer_part(self) -> Optional[Mixer]:
        raise NotImplementedError

    def forward(self, ctx: StepContext, stream: ResidualStream, cache: Optional[LayerCache],
                state: Optional[Dict[str, torch.Tensor]]) -> None:
        raise NotImplementedError
