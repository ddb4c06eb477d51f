"""The tiny models behind the golden files: configurations, token ids, the rows of the
logits that are stored, and weights drawn with numpy's PCG64 (a generator whose stream
does not change between versions) and rounded to float16, the precision of the
reference's tensor file (tools/model_exporter.py:168-171).  The head size is
hidden/heads, the only one the reference knows (src/libllm/llama.cc:117-120)."""
import hashlib
import os
import sys

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import plain_llama as P  # noqa: E402

CONFIG_A = dict(model_type="llama", num_hidden_layers=2, hidden_size=64, num_attention_heads=4,
                num_key_value_heads=2, head_dim=16, intermediate_size=192, vocab_size=256, rope_theta=10000.0,
                rope_scaling=None, rms_norm_eps=1e-5, tie_word_embeddings=True, max_position_embeddings=128)
CONFIG_B = dict(model_type="llama", num_hidden_layers=3, hidden_size=96, num_attention_heads=3,
                num_key_value_heads=1, head_dim=32, intermediate_size=256, vocab_size=512, rope_theta=500000.0,
                rope_scaling=dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                                  original_max_position_embeddings=64),
                rms_norm_eps=1e-6, tie_word_embeddings=False, max_position_embeddings=128)


def _ids(n, vocab, seed):
    return [int(v) for v in np.random.Generator(np.random.PCG64(seed)).integers(0, vocab, n)]


CASES = {
    "tiny_a": dict(config=CONFIG_A, seed=101, ids=_ids(12, 256, 7), rows=list(range(12))),
    "tiny_b": dict(config=CONFIG_B, seed=202, ids=_ids(70, 512, 8), rows=[0, 1, 6, 32, 33, 63, 64, 65, 69]),
}


def weights(c, seed):
    """Matrices N(0, 0.02), norm weights 1 + U(-0.1, 0.1), rounded to float16, as float32 tensors."""
    g = np.random.Generator(np.random.PCG64(seed))
    H, I, V = c["hidden_size"], c["intermediate_size"], c["vocab_size"]
    nH, nKV, d = c["num_attention_heads"], c["num_key_value_heads"], c["head_dim"]

    def mat(*shape):
        return torch.from_numpy((g.standard_normal(shape) * 0.02).astype(np.float16).astype(np.float32))

    def norm(n):
        return torch.from_numpy((1 + g.uniform(-0.1, 0.1, n)).astype(np.float16).astype(np.float32))
    w = {"model.embed_tokens.weight": mat(V, H)}
    for i in range(c["num_hidden_layers"]):
        p = f"model.layers.{i}."
        w[p + "input_layernorm.weight"] = norm(H)
        w[p + "self_attn.q_proj.weight"] = mat(nH * d, H)
        w[p + "self_attn.k_proj.weight"] = mat(nKV * d, H)
        w[p + "self_attn.v_proj.weight"] = mat(nKV * d, H)
        w[p + "self_attn.o_proj.weight"] = mat(H, nH * d)
        w[p + "post_attention_layernorm.weight"] = norm(H)
        w[p + "mlp.gate_proj.weight"] = mat(I, H)
        w[p + "mlp.up_proj.weight"] = mat(I, H)
        w[p + "mlp.down_proj.weight"] = mat(H, I)
    w["model.norm.weight"] = norm(H)
    if not c["tie_word_embeddings"]:
        w["lm_head.weight"] = mat(V, H)
    return w


def rope_table(c):
    """cos and sin, each [positions, d] with the d/2 angles repeated twice, rounded to float16
    as the reference stores them (src/libllm/llama.cc:282-283, tools/llama_exporter.py:54-62)."""
    f = P.rope_frequencies(c["head_dim"], c["rope_theta"], c["rope_scaling"])
    angle = torch.arange(c["max_position_embeddings"], dtype=torch.float64)[:, None] * f[None, :]
    cos = torch.cat([angle.cos(), angle.cos()], -1).to(torch.float16).to(torch.float32)
    sin = torch.cat([angle.sin(), angle.sin()], -1).to(torch.float16).to(torch.float32)
    return cos, sin


def checksum(w):
    h = hashlib.sha256()
    for k in sorted(w):
        h.update(k.encode())
        h.update(w[k].numpy().tobytes())
    return h.hexdigest()
