"""The plain implementation checked against itself: closed forms, hand-computed cases,
and the size of the bfloat16 rounding floor that the engine tests' bounds rest on."""
import math

import pytest
import torch

import plain_llama as P
from helpers import TINY, model_folder, plain_weights, rel_err, rms_err, tokens_for


def test_rms_norm_and_swiglu_by_hand():
    x = torch.tensor([[3.0, 4.0]])
    y = P.rms_norm(x, torch.tensor([2.0, 0.5]), 0.0)
    r = math.sqrt(12.5)
    assert torch.allclose(y, torch.tensor([[6.0 / r, 2.0 / r]], dtype=torch.float64))
    assert torch.allclose(P.swiglu(torch.tensor([0.0, 2.0]), torch.tensor([5.0, 3.0])),
                          torch.tensor([0.0, 2.0 / (1 + math.exp(-2.0)) * 3.0], dtype=torch.float64))


def test_rope_frequencies_llama3_has_all_three_branches():
    sc = TINY["B"]["rope_scaling"]
    base = P.rope_frequencies(32, 500000.0, None)
    f = P.rope_frequencies(32, 500000.0, sc)
    kept = [i for i in range(16) if f[i] == base[i]]
    scaled = [i for i in range(16) if abs(float(f[i]) - float(base[i]) / 8.0) < 1e-18]
    blended = [i for i in range(16) if i not in kept and i not in scaled]
    assert kept == [0, 1] and blended == [2] and scaled == list(range(3, 16))
    wl = 2 * math.pi / float(base[2])
    s = (64 / wl - 1.0) / (4.0 - 1.0)
    assert abs(float(f[2]) - ((1 - s) * float(base[2]) / 8 + s * float(base[2]))) < 1e-15


def test_rotation_keeps_lengths_and_depends_on_distance_only():
    g = torch.Generator().manual_seed(0)
    q, k = torch.randn(1, 1, 16, generator=g), torch.randn(1, 1, 16, generator=g)
    f = P.rope_frequencies(16, 10000.0, None)
    a = (P.rope_rotate(q, torch.tensor([7]), f) * P.rope_rotate(k, torch.tensor([3]), f)).sum()
    b = (P.rope_rotate(q, torch.tensor([104]), f) * P.rope_rotate(k, torch.tensor([100]), f)).sum()
    assert abs(float(a - b)) < 1e-12
    assert abs(float(P.rope_rotate(q, torch.tensor([9]), f).norm() - q.double().norm())) < 1e-12


def test_attention_mask_groups_and_window():
    g = torch.Generator().manual_seed(1)
    q, k, v = torch.randn(5, 4, 8, generator=g), torch.randn(5, 2, 8, generator=g), torch.randn(5, 2, 8, generator=g)
    out = P.attention_scores_softmax_values(q, k, v)
    assert torch.allclose(out[0, :, :], v[0, [0, 0, 1, 1], :].double())       # first token sees itself only
    s = (q[4, 3].double() @ k[:, 1].double().T) / math.sqrt(8)
    assert torch.allclose(out[4, 3], torch.softmax(s, 0) @ v[:, 1].double())
    # the last queries of a longer sequence: bottom-right alignment
    tail = P.attention_scores_softmax_values(q[3:], k, v)
    assert torch.allclose(tail, out[3:])
    w = P.attention_scores_softmax_values(q, k, v, window=2)
    s2 = (q[4, 0].double() @ k[3:5, 0].double().T) / math.sqrt(8)
    assert torch.allclose(w[4, 0], torch.softmax(s2, 0) @ v[3:5, 0].double())


def test_logits_of_a_prefix_do_not_depend_on_what_follows():
    for name in ("A", "B"):
        d = model_folder(name)
        c, w = P.read_config(d), plain_weights(d)
        t = tokens_for(name, 20, 3)
        assert torch.allclose(P.forward_logits(c, w, t)[:9], P.forward_logits(c, w, t[:9]), atol=1e-12)


def test_plain_sampler():
    logits = torch.tensor([1.0, 3.0, 2.0, 3.0, -1.0])
    assert P.sample_token(logits, 0.0, 0, 1.0, 0.3) == 1                       # greedy: first of the tied maxima
    assert P.sample_token(logits, 1.0, 1, 1.0, 0.99) == 1                      # top-1 is greedy
    p = torch.softmax(logits.double(), 0)
    # top_k 3 keeps tokens 1, 3, 2 in that order; top_p 0.5 cuts after the second
    assert P.sample_token(logits, 1.0, 3, 0.5, 0.49) == 1 and P.sample_token(logits, 1.0, 3, 0.5, 0.51) == 3
    assert P.sample_token(logits, 1.0, 3, 1.0, 0.999) == 2
    assert P.sample_token(logits, 1.0, 0, 1.0, float(p[0]) - 1e-9) == 0        # whole vocabulary, in index order
    assert P.sample_token(logits, 1.0, 0, 1.0, float(p[0]) + 1e-9) == 1
    with pytest.raises(IndexError):
        P.embedding(torch.zeros(4, 2), [4])


def test_bfloat16_rounding_floor():
    """How far the plain implementation moves when its activations are rounded to bfloat16
    where a bfloat16 engine has to round them: this is what the bounds of the engine tests
    are set against (tests/helpers.py)."""
    worst_max, worst_rms = 0.0, 0.0
    for name in ("A", "B", "C"):
        d = model_folder(name)
        c, w = P.read_config(d), plain_weights(d)
        t = tokens_for(name, 33, 3)
        exact, rounded = P.forward_logits(c, w, t), P.forward_logits(c, w, t, torch.bfloat16)
        worst_max = max(worst_max, rel_err(rounded, exact))
        worst_rms = max(worst_rms, rms_err(rounded, exact))
    assert 5e-3 < worst_max < 4e-2 and 1e-3 < worst_rms < 8e-3
