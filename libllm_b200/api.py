"""The Python entry point, in the manner of the reference's ``libllm`` package:
``Model(path, device)`` and ``model.complete(prompt, top_k, top_p, temperature)`` that
yields chunks as they are generated (python/libllm/__init__.py:56-111).  Prompts and
chunks are token ids: everything between a request's tokens and its next token is in
this library, text is not.  ``generate`` is the batched form the reference lacks."""
from __future__ import annotations

import queue
import threading
from dataclasses import dataclass
from enum import IntEnum
from typing import Iterable, Iterator, List, Optional, Sequence

from .engine.generate import generate as _generate
from .engine.model import Model as _Weights
from .engine.step import Engine, SamplingParams, StepItem
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
        weights = _Weights.from_folder(path, dtype=dtype, device=f"cuda:{cuda_device}",
                                       max_positions=max_seq_len)
        self._attach(weights, max_tokens, max_seq_len, use_graphs, max_step_tokens)
        self.path = path

    def _attach(self, weights, max_tokens, max_seq_len, use_graphs, max_step_tokens) -> None:
        self.weights = weights
        self.engine = Engine(weights, max_tokens=max_tokens, max_seq_len=max_seq_len,
                             use_graphs=use_graphs, max_step_tokens=max_step_tokens)
        self.path = None

    @classmethod
    def from_random(cls, config_json: dict, seed: int = 0, dtype: str = "bfloat16", max_tokens: int = 65536,
                    max_seq_len: Optional[int] = None, cuda_device: int = 0, use_graphs: bool = True,
                    max_step_tokens: int = 8192) -> "Model":
        """The random-weights mode without a folder: tensors are drawn on the device
        (matrices N(0, 0.02), norm weights 1 + U(-0.1, 0.1)) from ``seed``."""
        import torch
        from .config import architecture_for
        from .weights.random_model import random_tensors
        device = f"cuda:{cuda_device}"
        config = architecture_for(config_json["model_type"]).parse(config_json)
        tensors = random_tensors(config_json, seed, torch.bfloat16, device)
        self = cls.__new__(cls)
        self._attach(_Weights.from_tensors(config, tensors, dtype=dtype, device=device,
                                           max_positions=max_seq_len),
                     max_tokens, max_seq_len, use_graphs, max_step_tokens)
        return self

    @property
    def name(self) -> str:
        return self.weights.config.model_type

    @property
    def config(self):
        return self.weights.config

    def generate(self, prompts: Sequence[Sequence[int]], max_new_tokens=64, temperature: float = 1.0,
                 top_k: int = 50, top_p: float = 0.8, seed: int = 0,
                 stop_token_ids: Optional[Iterable[int]] = None, max_batch: int = 64,
                 on_token=None) -> List[List[int]]:
        """Tokens generated for each prompt (lists of token ids in, lists out).
        ``temperature=0`` is greedy; ``on_token(prompt index, token)`` is called as tokens arrive."""
        return _generate(self.engine, prompts, max_new_tokens, SamplingParams(temperature, top_k, top_p),
                         seed, stop_token_ids, max_batch, on_token)

    def complete(self, prompt: Sequence[int], top_k: int = 50, top_p: float = 0.8,
                 temperature: float = 1.0, max_new_tokens: int = 1 << 30, seed: int = 0) -> Iterator[Chunk]:
        """Completes one prompt, yielding a chunk per token until a stop token (the
        reference's defaults: python/libllm/__init__.py:75-76)."""
        room = self.engine.max_seq_len - len(prompt)
        limit = max(0, min(max_new_tokens, room))
        done = object()
        q: "queue.Queue" = queue.Queue()

        def work():
            try:
                _generate(self.engine, [list(prompt)], limit, SamplingParams(temperature, top_k, top_p),
                          seed, None, 1, on_token=lambda i, t: q.put(t))
                q.put(done)
            except BaseException as e:     # handed to the consumer
                q.put(e)

        t = threading.Thread(target=work, daemon=True)
        t.start()
        while True:
            item = q.get()
            if item is done:
                break
            if isinstance(item, BaseException):
                raise item
            yield Chunk(item)
        t.join()
