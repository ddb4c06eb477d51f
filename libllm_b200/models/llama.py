"""The Llama dense decoder as a ``ModelSpec``: which parts, which sizes, which tensors.

Layer structure and sizes follow the reference's build functions
(src/libllm/llama.cc:111-141, 231-249, 273-292); tensor names are the checkpoint's own,
the ones the reference's exporter reads them from (tools/llama_exporter.py:35-78)."""
from __future__ import annotations

from ..config import LlamaConfig, parse_llama_config, register_architecture
from ..parts.spec import (AttentionSpec, BlockSpec, ModelSpec, RMSNormSpec, RopeSpec, ScheduleEntry,
                          SwiGLUSpec)


def describe_llama(c: LlamaConfig) -> ModelSpec:
    rope = RopeSpec("rope", head_dim=c.head_dim, rotary_dim=c.head_dim, theta=c.rope_theta,
                    scaling=c.rope_scaling)
    layers = []
    for i in range(c.num_hidden_layers):
        p = f"model.layers.{i}."
        layers.append(BlockSpec(
            "prenorm",
            mixer_norm=RMSNormSpec("rmsnorm", c.hidden_size, c.rms_norm_eps, p + "input_layernorm.weight"),
            mixer=AttentionSpec("attention", hidden=c.hidden_size, n_heads=c.num_attention_heads,
                                n_kv_heads=c.num_key_value_heads, head_dim=c.head_dim, position=rope,
                                window=None, scale=None, bias=c.attention_bias,
                                q=p + "self_attn.q_proj.weight", k=p + "self_attn.k_proj.weight",
                                v=p + "self_attn.v_proj.weight", o=p + "self_attn.o_proj.weight"),
            ff_norm=RMSNormSpec("rmsnorm", c.hidden_size, c.rms_norm_eps, p + "post_attention_layernorm.weight"),
            ff=SwiGLUSpec("swiglu", hidden=c.hidden_size, intermediate=c.intermediate_size,
                          gate=p + "mlp.gate_proj.weight", up=p + "mlp.up_proj.weight",
                          down=p + "mlp.down_proj.weight"),
        ))
    return ModelSpec(
        vocab_size=c.vocab_size, hidden=c.hidden_size, embedding="model.embed_tokens.weight",
        layers=tuple(layers), schedule=tuple(ScheduleEntry(i) for i in range(c.num_hidden_layers)),
        final_norm=RMSNormSpec("rmsnorm", c.hidden_size, c.rms_norm_eps, "model.norm.weight"),
        head=None if c.tie_word_embeddings else "lm_head.weight",
        max_positions=c.max_position_embeddings, stop_tokens=c.eos_token_ids, name="llama")


register_architecture("llama", parse_llama_config, describe_llama, replace=True)
