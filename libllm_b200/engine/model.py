"""The generic model: a token table, the layers of a ``ModelSpec`` in the order of its
schedule, a last norm and the output matrix.  It knows parts and their interfaces, not
architectures; the architecture's name is used once, to look up the function that
describes it (libllm_b200/config/base.py)."""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..config import ModelConfig, architecture_for, load_config
from ..csrc import build, ops
from ..errors import ConfigError, InvalidArgError
from ..parts import fast
from ..parts.base import BuildEnv, CacheNeed, ResidualStream, StateNeed, StepContext
from ..parts.linear import linear
from ..parts.registry import build_part
from ..parts.spec import ModelSpec
from ..weights.state_map import StateMap, TensorNeed

DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16, torch.float32: torch.float32,
          torch.bfloat16: torch.bfloat16}


def resolve_dtype(dtype) -> torch.dtype:
    try:
        return DTYPES[dtype]
    except KeyError:
        raise InvalidArgError(f"dtype {dtype!r} is not supported (bfloat16 or float32)") from None


class Model:
    """Weights on the device plus the forward pass of one step.

    ``forward(ctx, cache)`` runs the tokens of ``ctx`` through every scheduled layer
    and returns 32-bit logits for ``ctx.want_rows`` (the reference computes logits of
    the last position only, src/libllm/llama.cc:353-354; its tests of all positions,
    src/libllm/llama_test.cc:92-97)."""

    def __init__(self, config: ModelConfig, spec: ModelSpec, dtype, device, max_positions: Optional[int] = None):
        self.config = config
        self.spec = spec
        self.dtype = resolve_dtype(dtype)
        self.device = torch.device(device)
        self.max_positions = min(max_positions or spec.max_positions, spec.max_positions)
        env = BuildEnv(self.dtype, self.device, self.max_positions)
        self.env = env
        self.layers = [build_part("block", b, env) for b in spec.layers]
        self.final_norm = build_part("norm", spec.final_norm, env)
        for i, e in enumerate(spec.schedule):
            if not 0 <= e.layer < len(self.layers):
                raise ConfigError(f"schedule entry {i} names layer {e.layer}, the model has {len(self.layers)}")
            if e.cache_from is not None and not 0 <= e.cache_from < i:
                raise ConfigError(f"schedule entry {i} reads the cache of entry {e.cache_from}, which does not run before it")
        self.embedding: Optional[torch.Tensor] = None
        self.head: Optional[torch.Tensor] = None

    # ---------------------------------------------------------------- weights
    def tensor_needs(self) -> List[TensorNeed]:
        s = self.spec
        needs = [TensorNeed(s.embedding, (s.vocab_size, s.hidden))]
        for layer in self.layers:
            needs.extend(layer.tensor_needs())
        needs.extend(self.final_norm.tensor_needs())
        if s.head is not None:
            needs.append(TensorNeed(s.head, (s.vocab_size, s.hidden)))
        return needs

    def load_state(self, state: StateMap) -> "Model":
        s = self.spec
        if self.device.type != "cuda":
            raise InvalidArgError("libllm_b200 runs on a CUDA device only (there is no CPU path)")
        needs = self.tensor_needs()
        # A tied checkpoint may still carry a copy of the output matrix; it is not used.
        allow = ["lm_head.weight"] if s.head is None else []
        state.check(needs, allow_unexpected=allow)

        def fetch(need: TensorNeed):
            return state.fetch(need, self.dtype, self.device)

        self.embedding = fetch(needs[0])
        for layer in self.layers:
            layer.load(fetch)
        self.final_norm.load(fetch)
        self.head = self.embedding if s.head is None else fetch(needs[-1])
        return self

    def kernel_families(self) -> List[str]:
        fams = {"elementwise", "sampling", *fast.product_families(self.dtype)}
        for layer in self.layers:
            fams.update(layer.kernel_families())
        return sorted(fams)

    @classmethod
    def from_folder(cls, folder: str, dtype="bfloat16", device="cuda:0",
                    max_positions: Optional[int] = None) -> "Model":
        config = load_config(folder)
        spec = architecture_for(config.model_type).describe(config)
        model = cls(config, spec, dtype, device, max_positions)
        build.ensure_built(model.kernel_families())
        state = StateMap.from_folder(folder)
        try:
            model.load_state(state)
        finally:
            state.close()
        return model

    @classmethod
    def from_tensors(cls, config: ModelConfig, tensors: Dict[str, torch.Tensor], dtype="bfloat16",
                     device="cuda:0", max_positions: Optional[int] = None) -> "Model":
        spec = architecture_for(config.model_type).describe(config)
        model = cls(config, spec, dtype, device, max_positions)
        build.ensure_built(model.kernel_families())
        return model.load_state(StateMap.from_tensors(tensors))

    # ---------------------------------------------------------------- what the cache must hold
    def run_cache_needs(self) -> List[Optional[CacheNeed]]:
        out = []
        for e in self.spec.schedule:
            mixer = self.layers[e.layer].mixer_part()
            out.append(mixer.cache_need() if (mixer is not None and e.cache_from is None) else None)
        return out

    def run_state_needs(self) -> List[Dict[str, StateNeed]]:
        out = []
        for e in self.spec.schedule:
            mixer = self.layers[e.layer].mixer_part()
            out.append(mixer.state_need() if mixer is not None else {})
        return out

    # ---------------------------------------------------------------- one step
    def forward(self, ctx: StepContext, cache, page_tables: List[torch.Tensor]) -> torch.Tensor:
        resid = torch.empty((ctx.n_tokens, self.spec.hidden), dtype=torch.float32, device=self.device)
        fed = ctx.extras.get("fed")          # (tokens of the previous step on the device, row per token)
        ops.embedding(self.embedding, ctx.tokens, resid, *(fed or ()))
        stream = ResidualStream(resid)
        for i, e in enumerate(self.spec.schedule):
            view = cache.layer_cache(i, e.cache_from, page_tables)
            self.layers[e.layer].forward(ctx, stream, view, cache.state[i] or None)
        h = self.final_norm.forward(ctx, stream, rows=ctx.want_rows)
        return linear(h, self.head, out_dtype=torch.float32)
