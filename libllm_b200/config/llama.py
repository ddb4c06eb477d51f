"""LlamaConfig: the typed configuration of the Llama dense decoder.

Fields are those the reference's loader reads (src/libllm/llama.cc:53-75) under the
names its exporter takes them from in config.json (tools/llama_exporter.py:90-100),
plus what the exporter resolves offline and this library resolves itself: the rotary
base and its "llama3" rescaling (the reference stores a finished table,
tools/llama_exporter.py:54-62), the head size, tied embeddings and the stop tokens."""
from __future__ import annotations

from dataclasses import dataclass, asdict
from typing import Any, Dict, Mapping, Optional, Tuple

from ..errors import ConfigError
from .base import ConfigReader, ModelConfig


@dataclass(frozen=True)
class RopeScaling:
    """The "llama3" frequency rescaling of config.json's ``rope_scaling``."""
    rope_type: str
    factor: float
    low_freq_factor: float
    high_freq_factor: float
    original_max_position_embeddings: int


@dataclass(frozen=True)
class LlamaConfig(ModelConfig):
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    vocab_size: int
    max_position_embeddings: int
    rms_norm_eps: float
    rope_theta: float
    rope_scaling: Optional[RopeScaling]
    tie_word_embeddings: bool
    attention_bias: bool
    eos_token_ids: Tuple[int, ...]
    bos_token_id: Optional[int]

    def to_json_dict(self) -> Dict[str, Any]:
        d = asdict(self)
        eos = d.pop("eos_token_ids")
        d["eos_token_id"] = list(eos) if len(eos) != 1 else eos[0]
        if not eos:
            d["eos_token_id"] = None
        d["hidden_act"] = "silu"
        return d


def parse_rope_scaling(raw, where: str) -> Optional[RopeScaling]:
    if raw is None:
        return None
    if not isinstance(raw, Mapping):
        raise ConfigError(f"{where}: 'rope_scaling' must be an object or null")
    kind = raw.get("rope_type", raw.get("type"))
    if kind in (None, "default"):
        return None
    if kind != "llama3":
        raise ConfigError(f"{where}: rope_scaling type '{kind}' is not supported (only 'llama3')")
    r = ConfigReader(raw, where + ": rope_scaling")
    s = RopeScaling("llama3", r.number("factor"), r.number("low_freq_factor"),
                    r.number("high_freq_factor"), r.integer("original_max_position_embeddings"))
    if s.high_freq_factor <= s.low_freq_factor:
        raise ConfigError(f"{where}: rope_scaling needs high_freq_factor > low_freq_factor")
    return s


def parse_llama_config(data: Mapping[str, Any]) -> LlamaConfig:
    """Checks follow the reference where it has them: hidden_size must divide by the
    number of heads when no head size is given ("invalid hidden_size and num_heads",
    src/libllm/llama.cc:117-118); the activation must be silu and pretraining_tp 1
    (tools/llama_exporter.py:87-88)."""
    where = "config.json"
    r = ConfigReader(data, where)
    hidden = r.integer("hidden_size")
    heads = r.integer("num_attention_heads")
    kv_heads = r.integer("num_key_value_heads", default=heads)
    head_dim = r.integer("head_dim", default=None)
    if head_dim is None:
        if hidden % heads != 0:
            raise ConfigError(f"{where}: invalid hidden_size and num_attention_heads "
                              f"({hidden} is not a multiple of {heads}) and no head_dim given")
        head_dim = hidden // heads
    if heads % kv_heads != 0:
        raise ConfigError(f"{where}: num_attention_heads ({heads}) must be a multiple of "
                          f"num_key_value_heads ({kv_heads})")
    if head_dim % 2 != 0:
        raise ConfigError(f"{where}: head_dim ({head_dim}) must be even for rotary pairs")
    act = r.string("hidden_act", default="silu")
    if act != "silu":
        raise ConfigError(f"{where}: hidden_act '{act}' is not supported (only 'silu')")
    if r.integer("pretraining_tp", default=1) != 1:
        raise ConfigError(f"{where}: pretraining_tp must be 1")
    if r.boolean("mlp_bias", default=False):
        raise ConfigError(f"{where}: mlp_bias is not supported")
    eos_raw = r.raw("eos_token_id")
    if eos_raw is None:
        eos: Tuple[int, ...] = ()
    elif isinstance(eos_raw, int) and not isinstance(eos_raw, bool):
        eos = (eos_raw,)
    elif isinstance(eos_raw, (list, tuple)) and all(isinstance(e, int) for e in eos_raw):
        eos = tuple(eos_raw)
    else:
        raise ConfigError(f"{where}: 'eos_token_id' must be an integer or a list of integers")
    vocab = r.integer("vocab_size")
    for e in eos:
        if not 0 <= e < vocab:
            raise ConfigError(f"{where}: eos_token_id {e} lies outside the vocabulary ({vocab})")
    return LlamaConfig(
        model_type=r.string("model_type"),
        hidden_size=hidden,
        num_hidden_layers=r.integer("num_hidden_layers"),
        num_attention_heads=heads,
        num_key_value_heads=kv_heads,
        head_dim=head_dim,
        intermediate_size=r.integer("intermediate_size"),
        vocab_size=vocab,
        max_position_embeddings=r.integer("max_position_embeddings"),
        rms_norm_eps=r.number("rms_norm_eps"),
        rope_theta=r.number("rope_theta", default=10000.0),
        rope_scaling=parse_rope_scaling(r.raw("rope_scaling"), where),
        tie_word_embeddings=r.boolean("tie_word_embeddings", default=False),
        attention_bias=r.boolean("attention_bias", default=False),
        eos_token_ids=eos,
        bos_token_id=r.integer("bos_token_id", default=None, minimum=0),
    )
