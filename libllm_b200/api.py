"""The Python entry point, in the manner of the reference's ``libllm`` package:
``Model(path, device)`` and ``model.complete(prompt, top_k, top_p, temperature)`` that
yields chunks as they are generated (python/libllm/__init__.py:56-111).  Prompts and
chunks are token ids: everything between a request's tokens and its next token is in
this library, text is not.  ``generate`` is the batched form the reference lacks.  Both run in
the host library (C++), as the reference's run in its own (python/libllm/interop.py:75-103)."""
from __future__ import annotations

from dataclasses import dataclass
from enum import IntEnum
from typing import Iterable, Iterator, List, Optional, Sequence

from .engine import Engine, SamplingParams
from .errors import InvalidArgError


class Device(IntEnum):
    """The reference's device codes (python/libllm/__init__.py:46-49).  Only CUDA exists
    here; AUTO means CUDA and CPU is refused."""
    CPU = 0x0000
    CUDA = 0x0100
    AUTO = 0x1f00


@dataclass
class Chunk:
    """One generated token (the reference's Chunk carries text, python/libllm/__init__.py:108-111)."""
    token: int

    @property
    def text(self) -> str:
        return f"<{self.token}>"


class Model:
    """A model folder (config.json + safetensors) loaded on one GPU, with its cache."""

    def __init__(self, path: str, device: Device = Device.AUTO, dtype: str = "bfloat16",
                 max_tokens: int = 65536, max_seq_len: Optional[int] = None, cuda_device: int = 0,
                 use_graphs: bool = True, max_step_tokens: int = 8192):
        if device == Device.CPU:
            raise InvalidArgError("this library has no CPU path: device must be CUDA or AUTO")
        self.engine = Engine.from_folder(path, dtype=dtype, max_tokens=max_tokens, max_seq_len=max_seq_len,
                                         max_step_tokens=max_step_tokens, use_graphs=use_graphs,
                                         cuda_device=cuda_device)
        self.path = path

    @classmethod
    def from_random(cls, config_json: dict, seed: int = 0, dtype: str = "bfloat16", max_tokens: int = 65536,
                    max_seq_len: Optional[int] = None, cuda_device: int = 0, use_graphs: bool = True,
                    max_step_tokens: int = 8192) -> "Model":
        """The random-weights mode without a folder: tensors are drawn on the device
        (matrices N(0, 0.02), norm weights 1 + U(-0.1, 0.1)) from ``seed``."""
        self = cls.__new__(cls)
        self.engine = Engine.from_random(config_json, seed, dtype=dtype, max_tokens=max_tokens, max_seq_len=max_seq_len,
                                         max_step_tokens=max_step_tokens, use_graphs=use_graphs,
                                         cuda_device=cuda_device)
        self.path = None
        return self

    @property
    def name(self) -> str:
        return self.engine.info()["name"]

    @property
    def config(self) -> dict:
        return self.engine.config

    def generate(self, prompts: Sequence[Sequence[int]], max_new_tokens=64, temperature: float = 1.0,
                 top_k: int = 50, top_p: float = 0.8, seed: int = 0,
                 stop_token_ids: Optional[Iterable[int]] = None, max_batch: int = 64,
                 on_token=None) -> List[List[int]]:
        """Tokens generated for each prompt (lists of token ids in, lists out).
        ``temperature=0`` is greedy; ``on_token(prompt index, token)`` is called as tokens arrive."""
        return self.engine.generate(prompts, max_new_tokens, SamplingParams(temperature, top_k, top_p), seed,
                                    stop_token_ids, max_batch, on_token)

    def complete(self, prompt: Sequence[int], top_k: int = 50, top_p: float = 0.8,
                 temperature: float = 1.0, max_new_tokens: int = 1 << 30, seed: int = 0) -> Iterator[Chunk]:
        """Completes one prompt, yielding a chunk per token until a stop token (the
        reference's defaults: python/libllm/__init__.py:75-76)."""
        for token in self.engine.complete(prompt, SamplingParams(temperature, top_k, top_p), max_new_tokens, seed):
            yield Chunk(token)
