"""The engine as Python sees it: a handle on the host library's model (weights, cache, step
function, graphs, generation loop), which is C++ (engine/step.cc, engine/generate.cc).  This
file converts arguments and results and nothing more."""
from __future__ import annotations

import ctypes
import json
from ctypes import c_float, c_int32, c_void_p
from dataclasses import dataclass
from typing import Any, Callable, Dict, Iterable, Iterator, List, Optional, Sequence, Tuple

import numpy as np

from .. import _lib
from ..errors import CacheError, EndOfSequence, InvalidArgError


@dataclass
class StepItem:
    """One sequence's share of a step: its slot, its next tokens, and the places among
    these tokens whose logits are wanted."""
    slot: int
    tokens: Sequence[int]
    want: Sequence[int] = ()
    fed_row: Optional[int] = None      # its one token is the one the previous step sampled for this row


@dataclass(frozen=True)
class SamplingParams:
    """temperature 0 is greedy; top_k 0 draws from the whole vocabulary.  The defaults
    are the reference's (src/libllm/llm.cc:125-132)."""
    temperature: float = 1.0
    top_k: int = 50
    top_p: float = 0.8

    def validate(self) -> None:
        _lib.check(_lib.lib().llm_validate_sampling(float(self.temperature), int(self.top_k), float(self.top_p)))

    def to_json(self) -> bytes:
        return json.dumps(dict(temperature=self.temperature, top_k=self.top_k, top_p=self.top_p)).encode()


GREEDY = SamplingParams(temperature=0.0, top_k=1, top_p=1.0)


def plan_batches(prompt_lengths: Sequence[int], max_new_tokens: Sequence[int], capacity_tokens: int,
                 max_batch: int, page_size: int = 64, max_seq_len: Optional[int] = None) -> List[List[int]]:
    """Splits requests, in order, into batches that fit the cache when every sequence grows to
    its full length (engine/generate.cc: plan_batches)."""
    out = _lib.Json()
    _lib.check(_lib.lib().llm_plan_batches(
        _lib.Json(dict(prompt_lengths=list(prompt_lengths), max_new_tokens=list(max_new_tokens),
                       capacity_tokens=capacity_tokens, max_batch=max_batch, page_size=page_size,
                       max_seq_len=max_seq_len or 0)).ref, out.ref))
    return out.get()


class PendingTokens:
    """Tokens of a step on their way from the device to the host."""

    def __init__(self, handle: c_void_p, n: int):
        self._h, self.n = handle, n

    def result(self) -> List[int]:
        buf = (c_int32 * max(1, self.n))()
        _lib.check(_lib.lib().llm_pending_result(ctypes.byref(self._h), buf))
        return list(buf[:self.n])

    def __del__(self):
        try:
            if self._h:
                _lib.lib().llm_pending_destroy(ctypes.byref(self._h))
        except Exception:
            pass


def _flatten(items: Sequence[StepItem]):
    slots, n_tok, toks, fed, n_want, want = [], [], [], [], [], []
    for it in items:
        slots.append(int(it.slot))
        n_tok.append(len(it.tokens))
        toks.extend(int(t) for t in it.tokens)
        fed.append(-1 if it.fed_row is None else int(it.fed_row))
        n_want.append(len(it.want))
        want.extend(int(w) for w in it.want)
    return slots, n_tok, toks, fed, n_want, want


class Engine:
    """A model on one GPU with its cache.  Make one with ``from_folder``, ``from_random`` or
    ``from_tensors``."""

    def __init__(self, handle: c_void_p, keep: Any = None):
        self._h = handle
        self._keep = keep
        self._info = None

    # ---------------------------------------------------------------- making one
    @staticmethod
    def _options(dtype, max_tokens, max_seq_len, max_slots, max_step_tokens, use_graphs, cuda_device, strict) -> Dict[str, Any]:
        kw: Dict[str, Any] = dict(dtype=str(dtype).replace("torch.", ""), max_tokens=int(max_tokens),
                                  max_step_tokens=int(max_step_tokens), use_graphs=bool(use_graphs),
                                  cuda_device=int(cuda_device), strict=bool(strict))
        if max_seq_len:
            kw["max_seq_len"] = int(max_seq_len)
        if max_slots:
            kw["max_slots"] = int(max_slots)
        return kw

    @classmethod
    def _load(cls, kw: Dict[str, Any], config_json: dict, loader: Callable[[c_void_p, _lib.Json], int], keep=None) -> "Engine":
        L = _lib.lib()
        _lib.use_families(_lib.describe_model(config_json, kw["dtype"])["kernel_families"])
        h = c_void_p()
        _lib.check(L.llm_model_init(ctypes.byref(h)))
        try:
            _lib.check(loader(h, _lib.Json(kw)))
        except Exception:
            L.llm_model_destroy(ctypes.byref(h))
            raise
        return cls(h, keep)

    @classmethod
    def from_folder(cls, folder: str, dtype="bfloat16", max_tokens: int = 65536, max_seq_len: Optional[int] = None,
                    max_slots: Optional[int] = None, max_step_tokens: int = 8192, use_graphs: bool = True,
                    cuda_device: int = 0, strict: bool = True, device: str = "auto") -> "Engine":
        import os
        kw = cls._options(dtype, max_tokens, max_seq_len, max_slots, max_step_tokens, use_graphs, cuda_device, strict)
        kw["filename"] = folder
        kw["device"] = device
        path = os.path.join(folder, "config.json")
        if not os.path.isfile(path):
            from ..errors import ConfigError
            raise ConfigError(f"{path}: no such file")
        with open(path) as f:
            try:
                config = json.load(f)
            except json.JSONDecodeError as e:
                from ..errors import ConfigError
                raise ConfigError(f"{path}: not valid JSON ({e})") from None
        return cls._load(kw, config, lambda h, j: _lib.lib().llm_model_load(ctypes.byref(h), j.ref))

    @classmethod
    def from_random(cls, config_json: dict, seed: int = 0, dtype="bfloat16", max_tokens: int = 65536,
                    max_seq_len: Optional[int] = None, max_slots: Optional[int] = None, max_step_tokens: int = 8192,
                    use_graphs: bool = True, cuda_device: int = 0) -> "Engine":
        """The random-weights mode without a folder: tensors are drawn on the device (matrices
        N(0, 0.02), norm weights 1 + U(-0.1, 0.1)) from ``seed``."""
        kw = cls._options(dtype, max_tokens, max_seq_len, max_slots, max_step_tokens, use_graphs, cuda_device, True)
        kw["random"] = dict(config=config_json, seed=int(seed))
        return cls._load(kw, config_json, lambda h, j: _lib.lib().llm_model_load(ctypes.byref(h), j.ref))

    @classmethod
    def from_tensors(cls, config_json: dict, tensors: Dict[str, Any], dtype="bfloat16", max_tokens: int = 65536,
                     max_seq_len: Optional[int] = None, max_slots: Optional[int] = None, max_step_tokens: int = 8192,
                     use_graphs: bool = True, cuda_device: int = 0, strict: bool = True) -> "Engine":
        """``tensors``: name -> numpy array (float32, float16, int32, ...) or torch tensor on the
        CPU (bfloat16 too).  They are read while this call runs and not kept."""
        kw = cls._options(dtype, max_tokens, max_seq_len, max_slots, max_step_tokens, use_graphs, cuda_device, strict)
        kw["config"] = config_json
        n, c_names, c_dtypes, c_shapes, c_ndims, c_ptrs, keep = _lib.host_tensors(tensors)

        def loader(h, j):
            return _lib.lib().llm_model_load_tensors(ctypes.byref(h), j.ref, n, c_names, c_dtypes, c_shapes, c_ndims, c_ptrs)
        return cls._load(kw, config_json, loader)

    # ---------------------------------------------------------------- what it is
    def info(self) -> Dict[str, Any]:
        out = _lib.Json()
        _lib.check(_lib.lib().llm_model_get_info(ctypes.byref(self._h), out.ref))
        return out.get()

    def _static(self) -> Dict[str, Any]:
        if self._info is None:
            self._info = self.info()
        return self._info

    @property
    def vocab(self) -> int:
        return self._static()["vocab_size"]

    @property
    def max_seq_len(self) -> int:
        return self._static()["max_seq_len"]

    @property
    def page_size(self) -> int:
        return self._static()["page_size"]

    @property
    def capacity_tokens(self) -> int:
        return self._static()["capacity_tokens"]

    @property
    def config(self) -> Dict[str, Any]:
        return self._static()["config"]

    @property
    def stop_tokens(self) -> List[int]:
        return self._static()["stop_tokens"]

    @property
    def stream(self) -> int:
        """The CUDA stream (its handle) that the engine's work is queued on."""
        s = c_void_p()
        _lib.check(_lib.lib().llm_model_stream(ctypes.byref(self._h), ctypes.byref(s)))
        return s.value or 0

    def cache_info(self) -> Dict[str, Any]:
        out = _lib.Json()
        _lib.check(_lib.lib().llm_model_cache_info(ctypes.byref(self._h), out.ref))
        return out.get()

    def cache_check(self) -> None:
        """Raises CacheError unless the cache's books are consistent (no page lost, held or freed twice)."""
        _lib.check(_lib.lib().llm_model_cache_check(ctypes.byref(self._h)))

    def pages_in_use(self) -> List[int]:
        return [g["pages_in_use"] for g in self.cache_info()["groups"]]

    # ---------------------------------------------------------------- sequences and steps
    def open_sequence(self) -> int:
        s = c_int32()
        _lib.check(_lib.lib().llm_model_open_sequence(ctypes.byref(self._h), ctypes.byref(s)))
        return s.value

    def close_sequence(self, slot: int) -> None:
        _lib.check(_lib.lib().llm_model_close_sequence(ctypes.byref(self._h), int(slot)))

    def sequence_length(self, slot: int) -> int:
        n = c_int32()
        _lib.check(_lib.lib().llm_model_sequence_length(ctypes.byref(self._h), int(slot), ctypes.byref(n)))
        return n.value

    def step(self, items: Sequence[StepItem], sampling: Optional[SamplingParams] = None,
             uniforms: Optional[Sequence[float]] = None, return_logits: bool = True):
        """Runs the items' tokens and returns the logits at the wanted places, float32
        [wanted, vocab] in the order of the items and of their ``want``.  With ``sampling`` it
        returns (logits or None, tokens): a token drawn at each wanted place; ``uniforms`` then
        holds one number in [0, 1) per wanted place."""
        items = list(items)
        slots, n_tok, toks, fed, n_want, want = _flatten(items)
        W = len(want)
        if sampling is not None and uniforms is not None and len(uniforms) != W:
            raise InvalidArgError("one uniform number per wanted place is needed")
        logits = np.empty((W, self.vocab), dtype=np.float32) if (return_logits or sampling is None) else None
        sampled = np.empty(max(W, 1), dtype=np.int32) if sampling is not None else None
        uni = None
        if sampling is not None and uniforms is not None:
            uni = (c_float * max(1, W))(*[float(u) for u in uniforms])
        _lib.check(_lib.lib().llm_model_step(
            ctypes.byref(self._h), len(items), _lib.int32_array(slots), _lib.int32_array(n_tok), _lib.int32_array(toks),
            _lib.int32_array(fed), _lib.int32_array(n_want), _lib.int32_array(want),
            sampling.to_json() if sampling is not None else None, uni,
            logits.ctypes.data_as(ctypes.POINTER(c_float)) if logits is not None else None,
            sampled.ctypes.data_as(ctypes.POINTER(c_int32)) if sampled is not None else None))
        if sampling is None:
            return logits
        return logits, sampled[:W]

    def step_tokens(self, items: Sequence[StepItem], sampling: SamplingParams,
                    uniforms: Optional[Sequence[float]] = None) -> PendingTokens:
        """Runs a step that samples one token per item (each wants exactly one place) and
        returns at once; the tokens stay on the device for the next step's ``fed_row``."""
        items = list(items)
        if any(len(it.want) != 1 for it in items):
            raise InvalidArgError("step_tokens: every item wants exactly one place")
        slots, n_tok, toks, fed, _, want = _flatten(items)
        uni = (c_float * max(1, len(items)))(*[float(u) for u in uniforms]) if uniforms is not None else None
        h = c_void_p()
        _lib.check(_lib.lib().llm_model_step_tokens(
            ctypes.byref(self._h), len(items), _lib.int32_array(slots), _lib.int32_array(n_tok), _lib.int32_array(toks),
            _lib.int32_array(fed), _lib.int32_array(want), sampling.to_json(), uni, ctypes.byref(h)))
        return PendingTokens(h, len(items))

    def synchronize(self) -> None:
        _lib.check(_lib.lib().llm_model_synchronize(ctypes.byref(self._h)))

    # ---------------------------------------------------------------- generation
    def generate(self, prompts: Sequence[Sequence[int]], max_new_tokens=64, sampling: SamplingParams = SamplingParams(),
                 seed: int = 0, stop_tokens: Optional[Iterable[int]] = None, max_batch: int = 64,
                 on_token: Optional[Callable[[int, int], None]] = None) -> List[List[int]]:
        """Generated tokens per prompt (engine/generate.cc).  ``max_new_tokens`` is one number or one
        per prompt; ``stop_tokens`` defaults to the model's own (config.json's eos_token_id);
        ``on_token(request index, token)`` is called as tokens arrive."""
        kw: Dict[str, Any] = dict(prompts=[[int(t) for t in p] for p in prompts],
                                  max_new_tokens=max_new_tokens if isinstance(max_new_tokens, int) else list(max_new_tokens),
                                  temperature=sampling.temperature, top_k=sampling.top_k, top_p=sampling.top_p,
                                  seed=int(seed), max_batch=int(max_batch))
        if stop_tokens is not None:
            kw["stop_token_ids"] = [int(t) for t in stop_tokens]
        cb, raised = None, []
        if on_token is not None:
            def relay(request, token, _user):
                try:
                    on_token(request, token)
                except BaseException as e:          # may not cross the C boundary
                    raised.append(e)
            cb = _TOKEN_FN(relay)
        out = _lib.Json()
        _lib.check(_lib.lib().llm_model_generate(ctypes.byref(self._h), _lib.Json(kw).ref,
                                                 ctypes.cast(cb, c_void_p) if cb else None, None, out.ref))
        if raised:
            raise raised[0]
        return out.get()["tokens"]

    def complete(self, prompt: Sequence[int], sampling: SamplingParams = SamplingParams(),
                 max_new_tokens: int = 1 << 30, seed: int = 0, stop_tokens: Optional[Iterable[int]] = None) -> Iterator[int]:
        """One prompt, token by token (the reference's completion handle, src/libllm/llm.cc:266-308)."""
        L = _lib.lib()
        kw: Dict[str, Any] = dict(prompt_ids=[int(t) for t in prompt], temperature=sampling.temperature, top_k=sampling.top_k,
                                  top_p=sampling.top_p, max_new_tokens=int(min(max_new_tokens, 1 << 30)), seed=int(seed))
        if stop_tokens is not None:
            kw["stop_token_ids"] = [int(t) for t in stop_tokens]
        comp = c_void_p()
        _lib.check(L.llm_completion_init(ctypes.byref(comp)))
        try:
            _lib.check(L.llm_model_complete(ctypes.byref(self._h), _lib.Json(kw).ref, ctypes.byref(comp)))
            chunk = _lib.Json()
            while True:
                try:
                    _lib.check(L.llm_completion_get_next_chunk(ctypes.byref(comp), chunk.ref))
                except EndOfSequence:
                    break
                yield int(chunk.get()["token"])
        finally:
            L.llm_completion_destroy(ctypes.byref(comp))

    # ---------------------------------------------------------------- test hooks
    def debug_set_status(self, code: int) -> None:
        _lib.check(_lib.lib().llm_model_debug_set_status(ctypes.byref(self._h), int(code)))

    def debug_wait_probe(self, limit_ns: int) -> None:
        _lib.check(_lib.lib().llm_model_debug_wait_probe(ctypes.byref(self._h), int(limit_ns)))

    def close(self) -> None:
        if self._h:
            _lib.lib().llm_model_destroy(ctypes.byref(self._h))
            self._h = c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


_TOKEN_FN = ctypes.CFUNCTYPE(None, c_int32, c_int32, c_void_p)


def generate(engine: Engine, prompts, max_new_tokens, sampling: SamplingParams = SamplingParams(), seed: int = 0,
             stop_tokens=None, max_batch: int = 64, on_token=None) -> List[List[int]]:
    return engine.generate(prompts, max_new_tokens, sampling, seed, stop_tokens, max_batch, on_token)


def should_stop(token: int, n_generated: int, max_new_tokens: int, stop_tokens) -> Tuple[bool, bool]:
    """(ends, emit), as engine/generate.cc decides it: a stop token ends the sequence and is not
    emitted; reaching the limit ends it after emitting.  (Asked of the library through a
    one-token plan so that the rule has one home.)"""
    out = _lib.Json()
    _lib.check(_lib.lib().llm_should_stop(int(token), int(n_generated), int(max_new_tokens),
                                          _lib.Json([int(t) for t in stop_tokens]).ref, out.ref))
    v = out.get()
    return bool(v["ends"]), bool(v["emit"])


__all__ = ["Engine", "GREEDY", "SamplingParams", "StepItem", "PendingTokens", "generate", "plan_batches", "should_stop"]
