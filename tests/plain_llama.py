"""Plain, slow implementation of the Llama decoder for tests.

Whole sequences, no cache, one function for each part, float64 by default so that it
is a reference for the 32-bit engine too.  It shares no code with the product path
(``libllm_b200``): it reads ``config.json`` itself and takes weights as a plain
``dict`` of tensors under their checkpoint names.

Every function restates a formula of ling0322/libllm and cites the file and lines
(paths are relative to that project's root).  Two things the reference does not
compute are restated from its exporter's inputs instead, and say so: the rotary
frequencies (the reference stores a ready-made cos/sin table,
``tools/llama_exporter.py:54-62``) and the choice between a tied and an untied output
matrix (the exporter always writes one, ``tools/llama_exporter.py:43``).
``tests/golden/`` holds outputs of the reference's own CPU code for the same tiny
model, against which this file is checked once.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional, Sequence

import torch

DT = torch.float64


def stored(x: torch.Tensor, act_dtype) -> torch.Tensor:
    """``x`` as it reads back after being stored in ``act_dtype`` (None: kept exact).

    A bfloat16 engine has to round an activation wherever a bfloat16 matrix product or the
    cache takes it: the outputs of the norms, q/k (after the rotation) and v, the attention
    output and the SwiGLU output.  With ``act_dtype=torch.bfloat16`` the plain
    implementation rounds at exactly these places and nowhere else, which gives the tests
    a reference that differs from a bfloat16 engine by accumulation order only."""
    return x if act_dtype is None else x.to(act_dtype).to(DT)


# ----------------------------------------------------------------------------- config
def read_config(folder: str) -> dict:
    """config.json as a plain dict with the defaults the reference's loader applies:
    ``num_key_value_heads`` falls back to the number of heads (src/libllm/llama.cc:64-68),
    the head size is hidden/heads unless given (src/libllm/llama.cc:117-120)."""
    with open(os.path.join(folder, "config.json")) as f:
        c = json.load(f)
    c.setdefault("num_key_value_heads", c["num_attention_heads"])
    if c.get("head_dim") is None:
        c["head_dim"] = c["hidden_size"] // c["num_attention_heads"]
    c.setdefault("rope_theta", 10000.0)
    c.setdefault("rope_scaling", None)
    c.setdefault("tie_word_embeddings", False)
    return c


# ----------------------------------------------------------------------------- parts
def embedding(table: torch.Tensor, ids: Sequence[int]) -> torch.Tensor:
    """x[t, :] = E[ids[t], :]  (src/flint/cpu/lookup.cc:33-57, src/libllm/layers.cc:36-47)."""
    for i in ids:
        if not 0 <= int(i) < table.shape[0]:
            raise IndexError(f"token id {i} outside the vocabulary of {table.shape[0]}")
    return table.to(DT)[torch.tensor(list(ids), dtype=torch.long)]


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """y = x * w / sqrt(mean(x^2) + eps) over the last axis; the weight multiplies
    directly, there is no ``1 + w`` (src/flint/cpu/normalizations.cc:52-64)."""
    x = x.to(DT)
    mean = (x * x).sum(-1, keepdim=True) / x.shape[-1]
    return x * weight.to(DT) / torch.sqrt(mean + eps)


def rope_frequencies(head_dim: int, theta: float, scaling: Optional[dict]) -> torch.Tensor:
    """Rotary frequencies f_i = theta^(-2i/d), i in [0, d/2), then the "llama3" rescaling.

    Not computed by the reference: its exporter stores the table that the checkpoint's
    rotary module returns (tools/llama_exporter.py:54-62; read at src/libllm/llama.cc:282-283).
    The llama3 rule as published with Llama 3.1: with wavelength L = 2*pi/f, frequencies
    with L < orig/high_freq_factor are kept, those with L > orig/low_freq_factor are
    divided by ``factor``, and between the two the result is the blend
    (1-s)*f/factor + s*f with s = (orig/L - low) / (high - low)."""
    i = torch.arange(0, head_dim // 2, dtype=DT)
    f = 1.0 / (float(theta) ** (2.0 * i / head_dim))
    if scaling is None:
        return f
    kind = scaling.get("rope_type", scaling.get("type"))
    if kind in (None, "default"):
        return f
    if kind != "llama3":
        raise ValueError(f"rope scaling {kind!r} is not part of this architecture")
    factor = float(scaling["factor"])
    low = float(scaling["low_freq_factor"])
    high = float(scaling["high_freq_factor"])
    orig = float(scaling["original_max_position_embeddings"])
    out = torch.empty_like(f)
    for j in range(f.numel()):
        fj = float(f[j])
        wavelen = 2.0 * math.pi / fj
        if wavelen < orig / high:
            out[j] = fj
        elif wavelen > orig / low:
            out[j] = fj / factor
        else:
            s = (orig / wavelen - low) / (high - low)
            out[j] = (1.0 - s) * fj / factor + s * fj
    return out


def rope_rotate(x: torch.Tensor, positions: torch.Tensor, freqs: torch.Tensor, table=None) -> torch.Tensor:
    """x*cos + rotate_half(x)*sin with rotate_half(x) = concat(-x[d/2:], x[:d/2]); cos and
    sin rows repeat the d/2 angles twice (src/libllm/llama.cc:151-176).  ``x`` is
    [tokens, heads, d], ``positions`` the absolute position of each token: the tokens
    already in the sequence come first (src/libllm/llama.cc:188-200).  ``table`` = (cos, sin),
    each [positions, d], replaces the computed angles: the reference reads such a table from
    its model file (src/libllm/llama.cc:282-283), and the golden test hands over the same one."""
    x = x.to(DT)
    if table is not None:
        cos = table[0].to(DT)[positions.long()][:, None, :]
        sin = table[1].to(DT)[positions.long()][:, None, :]
    else:
        angle = positions.to(DT)[:, None] * freqs[None, :]          # [T, d/2]
        cos = torch.cat([angle.cos(), angle.cos()], dim=-1)[:, None, :]
        sin = torch.cat([angle.sin(), angle.sin()], dim=-1)[:, None, :]
    half = x.shape[-1] // 2
    rotated = torch.cat([-x[..., half:], x[..., :half]], dim=-1)
    return x * cos + rotated * sin


def attention_scores_softmax_values(q, k, v, window: Optional[int] = None) -> torch.Tensor:
    """Causal grouped-query attention over a whole sequence.

    q [T, nH, d], k and v [S, nKV, d] with S >= T; query t stands at absolute position
    S-T+t and sees keys j <= S-T+t (mask aligned to the bottom right,
    src/flint/operators.cc:119-124).  Query head h reads key/value head
    h // (nH/nKV) (src/flint/operators.cc:43-56).  The scale sqrt(1/sqrt(d)) is applied
    to q and to k, 1/sqrt(d) in all (src/flint/operators.cc:115-117); softmax over keys,
    then the weighted sum of values (src/flint/operators.cc:126).
    ``window`` (not an option of this architecture; kept for parts that have one) limits
    query at position p to keys j > p - window."""
    T, nH, d = q.shape
    S, nKV, _ = k.shape
    group = nH // nKV
    scale = math.sqrt(1.0 / math.sqrt(d))
    out = torch.empty(T, nH, d, dtype=DT)
    qpos = torch.arange(S - T, S)
    kpos = torch.arange(S)
    allowed = kpos[None, :] <= qpos[:, None]
    if window is not None:
        allowed &= kpos[None, :] > (qpos[:, None] - window)
    for h in range(nH):
        kh = k[:, h // group, :].to(DT) * scale
        vh = v[:, h // group, :].to(DT)
        s = (q[:, h, :].to(DT) * scale) @ kh.T                  # [T, S]
        s = s.masked_fill(~allowed, float("-inf"))
        p = torch.softmax(s, dim=-1)
        out[:, h, :] = p @ vh
    return out


def linear(x: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y = x @ W^T (+ b); weights are [out, in] (src/libllm/layers.cc:79-92)."""
    y = x.to(DT) @ w.to(DT).T
    return y if b is None else y + b.to(DT)


def attention_block(x, positions, w: Dict[str, torch.Tensor], prefix: str, c: dict,
                    window: Optional[int] = None, act_dtype=None) -> torch.Tensor:
    """q, k, v projections, rotation of q and k, attention, output projection
    (src/libllm/llama.cc:178-225).  The reference multiplies by one stacked matrix
    [Wq; Wk; Wv] and slices (src/libllm/llama.cc:180-186, tools/llama_exporter.py:64-71);
    three products with the separate matrices are the same numbers."""
    nH, nKV, d = c["num_attention_heads"], c["num_key_value_heads"], c["head_dim"]
    T = x.shape[0]
    q = linear(x, w[prefix + "q_proj.weight"], w.get(prefix + "q_proj.bias")).view(T, nH, d)
    k = linear(x, w[prefix + "k_proj.weight"], w.get(prefix + "k_proj.bias")).view(T, nKV, d)
    v = linear(x, w[prefix + "v_proj.weight"], w.get(prefix + "v_proj.bias")).view(T, nKV, d)
    freqs = rope_frequencies(d, c["rope_theta"], c["rope_scaling"])
    q = stored(rope_rotate(q, positions, freqs, c.get("rope_table")), act_dtype)
    k = stored(rope_rotate(k, positions, freqs, c.get("rope_table")), act_dtype)
    v = stored(v, act_dtype)
    o = stored(attention_scores_softmax_values(q, k, v, window), act_dtype)
    return linear(o.reshape(T, nH * d), w[prefix + "o_proj.weight"])


def swiglu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """silu(gate) * up with silu(a) = a / (1 + exp(-a)); the gate is the first half of the
    stacked product, up the second (src/flint/cpu/swiglu.cc:49-54, tools/llama_exporter.py:73-77)."""
    gate = gate.to(DT)
    return gate * (1.0 / (1.0 + torch.exp(-gate))) * up.to(DT)


def feed_forward(x, w: Dict[str, torch.Tensor], prefix: str, act_dtype=None) -> torch.Tensor:
    """down(swiglu(gate(x), up(x))), no biases (src/libllm/llama.cc:81-98)."""
    g = linear(x, w[prefix + "gate_proj.weight"])
    u = linear(x, w[prefix + "up_proj.weight"])
    return linear(stored(swiglu(g, u), act_dtype), w[prefix + "down_proj.weight"])


def decoder_layer(x, positions, w, i: int, c: dict, act_dtype=None) -> torch.Tensor:
    """Pre-norm residual block: x + attn(norm(x)), then h + mlp(norm(h))
    (src/libllm/llama.cc:251-267)."""
    p = f"model.layers.{i}."
    eps = c["rms_norm_eps"]
    h = x + attention_block(stored(rms_norm(x, w[p + "input_layernorm.weight"], eps), act_dtype), positions,
                            w, p + "self_attn.", c, None, act_dtype)
    return h + feed_forward(stored(rms_norm(h, w[p + "post_attention_layernorm.weight"], eps), act_dtype), w,
                            p + "mlp.", act_dtype)


def forward_logits(c: dict, w: Dict[str, torch.Tensor], ids: Sequence[int], act_dtype=None,
                   rows: Optional[Sequence[int]] = None) -> torch.Tensor:
    """Logits at every position (or at ``rows``) of one whole sequence, [T, vocab], float64: embedding,
    the layers in order, the last norm (src/libllm/llama.cc:294-303), then the output
    matrix (src/libllm/llama.cc:305-308), which is the embedding table when
    ``tie_word_embeddings`` is set (the exporter writes the checkpoint's lm_head, which
    is that same table for a tied checkpoint: tools/llama_exporter.py:43)."""
    x = embedding(w["model.embed_tokens.weight"], ids)
    positions = torch.arange(len(ids))
    for i in range(c["num_hidden_layers"]):
        x = decoder_layer(x, positions, w, i, c, act_dtype)
    if rows is not None:
        x = x[list(rows)]
    x = stored(rms_norm(x, w["model.norm.weight"], c["rms_norm_eps"]), act_dtype)
    head = w["model.embed_tokens.weight"] if c["tie_word_embeddings"] else w["lm_head.weight"]
    return linear(x, head)


# ----------------------------------------------------------------------------- sampling
def sample_token(logits: torch.Tensor, temperature: float, top_k: int, top_p: float,
                 u: float) -> int:
    """One draw as the reference's sampler makes it: logits/temperature
    (src/libllm/generator.cc:200-203), softmax (:205), the ``top_k`` most probable in
    falling order (:65-89), the shortest prefix of them whose probabilities reach
    ``top_p`` (:47-63), then r = u * (their sum) and the first candidate whose running
    sum exceeds r (:91-111).  ``temperature == 0`` is greedy (lowest index on ties), and
    ``top_k == 0`` means every token is a candidate, in the vocabulary's order; neither
    exists in the reference."""
    logits = logits.to(DT)
    if temperature == 0:
        return int(torch.argmax(logits))   # first maximal index
    p = torch.softmax(logits / temperature, dim=-1)
    if top_k == 0:
        acc = torch.cumsum(p, 0)
        r = u * float(acc[-1])
        idx = int(torch.searchsorted(acc, torch.tensor(r, dtype=DT), right=True))
        return min(idx, p.numel() - 1)
    k = min(top_k, p.numel())
    order = sorted(range(p.numel()), key=lambda j: (-float(p[j]), j))[:k]
    chosen: List[int] = []
    total = 0.0
    for j in order:
        chosen.append(j)
        total += float(p[j])
        if total >= top_p:
            break
    r = u * total
    acc = 0.0
    for j in chosen:
        acc += float(p[j])
        if r < acc:
            return j
    return chosen[-1]


def greedy_continuation(c: dict, w: Dict[str, torch.Tensor], prompt: Sequence[int], n_new: int,
                        stop: Sequence[int] = ()) -> List[int]:
    """Greedy decoding by running the whole sequence again for every token.  As in the
    reference's loop a stop token ends the sequence and is not returned
    (src/libllm/generator.cc:140-156)."""
    ids = list(prompt)
    out: List[int] = []
    for _ in range(n_new):
        nxt = int(torch.argmax(forward_logits(c, w, ids)[-1]))
        if nxt in stop:
            break
        out.append(nxt)
        ids.append(nxt)
    return out
