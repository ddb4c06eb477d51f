"""The engine at the layer sizes of the models the benchmark names (Llama-3.2-1B, 3.2-3B, 3.1-8B:
head sizes 64 and 128, groups of 4 and 3, widths 2048 to 4096), with two layers and a small
vocabulary so that the plain implementation stays affordable: a prompt in one step, then tokens one
by one, in an unequal batch, in bfloat16 (the fast kernels) and float32."""
import pytest
import torch

import plain_llama as P
from helpers import TOL, model_folder, plain_weights, rel_err, rms_err
from replay import replay_batch

pytestmark = pytest.mark.gpu


def sized(hidden, heads, kv_heads, head_dim, inter, factor):
    return dict(model_type="llama", num_hidden_layers=2, hidden_size=hidden, num_attention_heads=heads,
                num_key_value_heads=kv_heads, head_dim=head_dim, intermediate_size=inter, vocab_size=1000,
                rope_theta=500000.0,
                rope_scaling=dict(rope_type="llama3", factor=factor, low_freq_factor=1.0, high_freq_factor=4.0,
                                  original_max_position_embeddings=8192),
                rms_norm_eps=1e-5, tie_word_embeddings=hidden != 4096, max_position_embeddings=4096,
                hidden_act="silu")


SIZES = {
    "1b": sized(2048, 32, 8, 64, 8192, 32.0),
    "3b": sized(3072, 24, 8, 128, 8192, 32.0),
    "8b": sized(4096, 32, 8, 128, 14336, 8.0),
}
_plain = {}


def reference(name, folder, toks, act_dtype=None):
    key = (name, tuple(toks), act_dtype)
    if key not in _plain:
        _plain[key] = P.forward_logits(P.read_config(folder), plain_weights(folder), toks, act_dtype=act_dtype)
    return _plain[key]


def check_float32(got, name, folder, toks, what):
    """float32: the engine adds each sum of K products in 32-bit (unit roundoff 6e-8), and such a sum's
    error grows with sqrt(K).  helpers.TOL was set on models whose longest sum has 256 terms; here the
    longest has 8,192 or 14,336 (the feed-forward's width), so the bounds scale by sqrt(K / 256).  A
    fault shows as 1e-3 or more; measured here: 2.0e-5, 3.5e-5 and 3.7e-5 at the three sizes."""
    c = SIZES[name]
    longest = max(c["hidden_size"], c["intermediate_size"], c["num_attention_heads"] * c["head_dim"])
    scale = (longest / 256) ** 0.5
    exact = reference(name, folder, toks)
    e, r = rel_err(got, exact), rms_err(got, exact)
    assert torch.isfinite(got).all()
    assert e < TOL["float32"][0] * scale, f"{what}: rel err {e:.3e} exceeds {TOL['float32'][0] * scale:.1e}"
    assert r < TOL["float32"][1] * scale, f"{what}: rms err {r:.3e} exceeds {TOL['float32'][1] * scale:.1e}"
    assert torch.equal(got.cpu().argmax(-1), exact.argmax(-1)) or \
        bool(((got.cpu().argmax(-1) == exact.argmax(-1)) |
              ((exact.topk(2, -1).values[..., 0] - exact.topk(2, -1).values[..., 1]) < 1e-3 * float(exact.abs().mean()))).all())


def check_against_the_floor(got, name, folder, toks, what):
    """bfloat16 at these widths: the bound is twice the distance between the plain implementation
    with activations rounded to bfloat16 where an engine must round them and its exact form, measured
    here for this model (the tiny models' bound in helpers.TOL was found the same way)."""
    exact = reference(name, folder, toks)
    rounded = reference(name, folder, toks, torch.bfloat16)
    floor_max, floor_rms = rel_err(rounded, exact), rms_err(rounded, exact)
    e, r = rel_err(got, exact), rms_err(got, exact)
    assert torch.isfinite(got).all()
    assert e < 2 * floor_max, f"{what}: rel err {e:.3e}, the rounding floor is {floor_max:.3e}"
    assert r < 2 * floor_rms, f"{what}: rms err {r:.3e}, the rounding floor is {floor_rms:.3e}"
    top2 = exact.topk(2, dim=-1).values
    clear = (top2[..., 0] - top2[..., 1]) > 4 * floor_max * float(exact.abs().mean())
    assert bool(((got.cpu().argmax(-1) == exact.argmax(-1)) | ~clear).all()), f"{what}: argmax differs where the margin is clear"


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
@pytest.mark.parametrize("name", sorted(SIZES))
def test_layer_sizes_of_the_benchmark_models(name, dtype):
    from libllm_b200.engine import Engine
    folder = model_folder("size_" + name, seed=9, config=SIZES[name])
    engine = Engine.from_folder(folder, dtype=dtype, max_tokens=512, max_seq_len=256)
    g = torch.Generator().manual_seed(3)
    long_ = torch.randint(0, 1000, (70,), generator=g).tolist()
    short = torch.randint(0, 1000, (9,), generator=g).tolist()
    got = replay_batch(engine, [("long", long_, 66), ("short", short, 3)])
    for rid, toks in (("long", long_), ("short", short)):
        if dtype == "float32":
            check_float32(got[rid], name, folder, toks, f"{name} {rid}")
        else:
            check_against_the_floor(got[rid], name, folder, toks, f"{name} {rid}")
    engine.close()


@pytest.mark.parametrize("name,n_prompt", [("3b", 300), ("8b", 257)])
def test_a_long_prompt_at_head_size_128(name, n_prompt):
    """Prompts of more than 128 tokens at head size 128 take the prompt attention's form with 256
    query rows a CTA: here through the engine (the kernel tests call both forms directly), with a
    prompt that ends inside a query tile and inside a key tile, beside a short one."""
    from libllm_b200.engine import Engine
    folder = model_folder("size_" + name, seed=9, config=SIZES[name])
    engine = Engine.from_folder(folder, dtype="bfloat16", max_tokens=1024, max_seq_len=512)
    g = torch.Generator().manual_seed(4)
    long_ = torch.randint(0, 1000, (n_prompt + 3,), generator=g).tolist()
    short = torch.randint(0, 1000, (140,), generator=g).tolist()
    got = replay_batch(engine, [("long", long_, n_prompt), ("short", short, 137)])
    for rid, toks in (("long", long_), ("short", short)):
        check_against_the_floor(got[rid], name, folder, toks, f"{name} {rid}")
    engine.close()
