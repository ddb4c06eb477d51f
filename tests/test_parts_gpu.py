"""Each part a layer is put together from, built from its spec and run alone against the
plain implementation's function for it, at sizes other than the tiny models'."""

import pytest
import torch

import plain_llama as P
from helpers import TOL, rel_err

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]
PAGE = 64


def env_for(dtype, max_positions=512):
    from libllm_b200.csrc import build
    from libllm_b200.parts.base import BuildEnv
    build.ensure_built()
    return BuildEnv(getattr(torch, dtype), torch.device("cuda:0"), max_positions)


def loader(weights, dtype):
    """The ``fetch`` a model hands its parts, over a plain dict."""
    from libllm_b200.weights.state_map import StateMap
    state = StateMap.from_tensors(weights)
    return lambda need: state.fetch(need, getattr(torch, dtype), "cuda:0")


def make_context(q_lens, past_lens, dtype, vocab=100, seed=0):
    """A step's description built by hand: sequences of ``q_lens`` new tokens behind
    ``past_lens`` cached ones, every sequence with pages of its own."""
    from libllm_b200.parts.base import StepContext
    dev = torch.device("cuda:0")
    B, T = len(q_lens), sum(q_lens)
    g = torch.Generator().manual_seed(seed)
    tokens = torch.randint(0, vocab, (T,), generator=g).to(torch.int32)
    tok_seq = torch.cat([torch.full((n,), b, dtype=torch.int32) for b, n in enumerate(q_lens)])
    tok_pos = torch.cat([torch.arange(p, p + n, dtype=torch.int32) for n, p in zip(q_lens, past_lens)])
    starts = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32)
    width = max((p + n + PAGE - 1) // PAGE for n, p in zip(q_lens, past_lens))
    # pages handed out in a scattered order: sequence b's logical page j is page j * B + b
    table = torch.tensor([[j * B + b for j in range(width)] for b in range(B)], dtype=torch.int32)
    ctx = StepContext(dtype=getattr(torch, dtype), device=dev, n_tokens=T, n_seqs=B, tokens=tokens.to(dev),
                      tok_seq=tok_seq.to(dev), tok_pos=tok_pos.to(dev), seq_start=starts.to(dev),
                      seq_past=torch.tensor(past_lens, dtype=torch.int32, device=dev),
                      seq_slot=torch.arange(B, dtype=torch.int32, device=dev),
                      want_rows=torch.arange(T, dtype=torch.int32, device=dev), q_lens=list(q_lens),
                      past_lens=list(past_lens), slots=list(range(B)), max_q_len=max(q_lens),
                      max_kv_len=max(p + n for n, p in zip(q_lens, past_lens)),
                      decode_only=all(n == 1 for n in q_lens))
    return ctx, table.to(dev), width * B


def close(got, ref, dtype, what):
    e = rel_err(got, ref)
    assert e < TOL[dtype][0], f"{what}: rel err {e:.3e} ({dtype})"


@pytest.mark.parametrize("dtype", DTYPES)
def test_rmsnorm_part_applies_the_pending_addition(dtype):
    from libllm_b200.parts.base import ResidualStream
    from libllm_b200.parts.registry import build_part
    from libllm_b200.parts.spec import RMSNormSpec
    H, eps = 104, 3e-4
    w = {"n.weight": 1 + 0.1 * torch.randn(H)}
    part = build_part("norm", RMSNormSpec("rmsnorm", H, eps, "n.weight"), env_for(dtype))
    part.load(loader(w, dtype))
    ctx, _, _ = make_context([5, 2], [0, 0], dtype)
    resid = torch.randn(7, H, device="cuda")
    pending = torch.randn(7, H, device="cuda")
    stream = ResidualStream(resid.clone())
    stream.pending = pending.clone()
    got = part.forward(ctx, stream)
    assert stream.pending is None
    assert torch.equal(stream.resid, resid + pending)            # the stream itself moves on, in 32-bit
    ref = P.rms_norm((resid + pending).cpu(), w["n.weight"], eps)
    close(got, ref, dtype, "rmsnorm part")
    # a subset of rows (the last norm before the output matrix) leaves the stream alone
    rows = torch.tensor([6, 1], dtype=torch.int32, device="cuda")
    before = stream.resid.clone()
    got = part.forward(ctx, stream, rows=rows)
    assert torch.equal(stream.resid, before)
    close(got, ref[[6, 1]], dtype, "rmsnorm part, chosen rows")


def test_rope_part_holds_the_table_of_the_plain_frequencies():
    from libllm_b200.config.llama import RopeScaling
    from libllm_b200.parts.registry import build_part
    from libllm_b200.parts.spec import RopeSpec
    sc = dict(rope_type="llama3", factor=4.0, low_freq_factor=1.0, high_freq_factor=8.0,
              original_max_position_embeddings=128)
    spec = RopeSpec("rope", head_dim=48, rotary_dim=48, theta=30000.0, scaling=RopeScaling(**sc))
    part = build_part("position", spec, env_for("float32", max_positions=300))
    part.load(None)
    f = P.rope_frequencies(48, 30000.0, sc)
    angle = torch.arange(300, dtype=torch.float64)[:, None] * f[None, :]
    ref = torch.cat([angle.cos(), angle.sin()], 1)
    assert tuple(part.table.shape) == (300, 48)
    assert float((part.table.cpu().double() - ref).abs().max()) < 1e-6


def attention_weights(H, nH, nKV, d, seed=0):
    g = torch.Generator().manual_seed(seed)
    r = lambda *s: (torch.randn(*s, generator=g) * 0.08).to(torch.bfloat16).float()
    return {"a.q_proj.weight": r(nH * d, H), "a.k_proj.weight": r(nKV * d, H), "a.v_proj.weight": r(nKV * d, H),
            "a.o_proj.weight": r(H, nH * d)}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,nH,nKV,d,window", [(72, 6, 2, 16, None), (40, 5, 5, 32, None), (64, 2, 1, 48, 37)])
def test_attention_part_prompt_then_single_tokens(dtype, H, nH, nKV, d, window):
    """The mixer alone: a prompt in one call, then tokens one by one, against the plain
    attention over the whole sequence; two sequences of unequal lengths share the calls."""
    from libllm_b200.parts.base import LayerCache
    from libllm_b200.parts.registry import build_part
    from libllm_b200.parts.spec import AttentionSpec, RopeSpec
    tdt = getattr(torch, dtype)
    w = attention_weights(H, nH, nKV, d)
    spec = AttentionSpec("attention", hidden=H, n_heads=nH, n_kv_heads=nKV, head_dim=d,
                         position=RopeSpec("rope", head_dim=d, rotary_dim=d, theta=10000.0, scaling=None),
                         window=window, q="a.q_proj.weight", k="a.k_proj.weight", v="a.v_proj.weight",
                         o="a.o_proj.weight")
    part = build_part("mixer", spec, env_for(dtype))
    part.load(loader(w, dtype))
    need = part.cache_need()
    assert (need.n_kv_heads, need.head_dim, need.window) == (nKV, d, window)
    lens = [70, 9]
    total = [lens[0] + 3, lens[1] + 3]
    g = torch.Generator().manual_seed(5)
    xs = [torch.randn(n, H, generator=g).to(torch.bfloat16).float() for n in total]
    c = dict(num_attention_heads=nH, num_key_value_heads=nKV, head_dim=d, rope_theta=10000.0, rope_scaling=None)
    refs = [P.attention_block(x, torch.arange(x.shape[0]), w, "a.", c, window) for x in xs]
    kc = vc = None
    outs = [[], []]
    for step in range(4):
        q_lens = lens if step == 0 else [1, 1]
        past = [0, 0] if step == 0 else [lens[0] + step - 1, lens[1] + step - 1]
        ctx, table, n_pages = make_context(q_lens, past, dtype)
        if kc is None:
            kc = torch.zeros(n_pages + 8, nKV, PAGE, d, dtype=tdt, device="cuda")
            vc = torch.zeros_like(kc)
        x = torch.cat([xs[b][past[b]:past[b] + q_lens[b]] for b in range(2)]).to(tdt).cuda()
        out = part.forward(ctx, x, LayerCache(kc, vc, table, PAGE, True), None)
        if out.dim() == 3:
            out = out.sum(0)
        o = 0
        for b in range(2):
            outs[b].append(out[o:o + q_lens[b]].float().cpu())
            o += q_lens[b]
    for b in range(2):
        close(torch.cat(outs[b]), refs[b], dtype, f"attention part, sequence {b}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T,H,I", [(1, 40, 104), (37, 72, 200)])
def test_swiglu_part(dtype, T, H, I):
    from libllm_b200.parts.registry import build_part
    from libllm_b200.parts.spec import SwiGLUSpec
    g = torch.Generator().manual_seed(1)
    r = lambda *s: (torch.randn(*s, generator=g) * 0.1).to(torch.bfloat16).float()
    w = {"m.gate_proj.weight": r(I, H), "m.up_proj.weight": r(I, H), "m.down_proj.weight": r(H, I)}
    part = build_part("feed_forward", SwiGLUSpec("swiglu", hidden=H, intermediate=I, gate="m.gate_proj.weight",
                                                 up="m.up_proj.weight", down="m.down_proj.weight"), env_for(dtype))
    part.load(loader(w, dtype))
    ctx, _, _ = make_context([T], [0], dtype)
    x = r(T, H)
    out = part.forward(ctx, x.to(getattr(torch, dtype)).cuda())
    if out.dim() == 3:
        out = out.sum(0)
    close(out, P.feed_forward(x, w, "m."), dtype, "swiglu part")


@pytest.mark.parametrize("dtype", DTYPES)
def test_prenorm_block_alone(dtype):
    """A whole layer from its spec against the plain layer: the block adds nothing of
    its own to what its parts compute, and leaves the last addition pending."""
    from libllm_b200.parts.base import LayerCache, ResidualStream
    from libllm_b200.parts.registry import build_part
    from libllm_b200.parts.spec import AttentionSpec, BlockSpec, RMSNormSpec, RopeSpec, SwiGLUSpec
    H, nH, nKV, d, I, eps = 48, 3, 3, 16, 88, 2e-5
    tdt = getattr(torch, dtype)
    g = torch.Generator().manual_seed(2)
    r = lambda *s: (torch.randn(*s, generator=g) * 0.1).to(torch.bfloat16).float()
    p = "model.layers.0."
    w = {p + "self_attn.q_proj.weight": r(nH * d, H), p + "self_attn.k_proj.weight": r(nKV * d, H),
         p + "self_attn.v_proj.weight": r(nKV * d, H), p + "self_attn.o_proj.weight": r(H, nH * d),
         p + "mlp.gate_proj.weight": r(I, H), p + "mlp.up_proj.weight": r(I, H), p + "mlp.down_proj.weight": r(H, I),
         p + "input_layernorm.weight": 1 + r(H), p + "post_attention_layernorm.weight": 1 + r(H)}
    spec = BlockSpec(
        "prenorm", mixer_norm=RMSNormSpec("rmsnorm", H, eps, p + "input_layernorm.weight"),
        mixer=AttentionSpec("attention", hidden=H, n_heads=nH, n_kv_heads=nKV, head_dim=d,
                            position=RopeSpec("rope", head_dim=d, rotary_dim=d, theta=1e4, scaling=None),
                            q=p + "self_attn.q_proj.weight", k=p + "self_attn.k_proj.weight",
                            v=p + "self_attn.v_proj.weight", o=p + "self_attn.o_proj.weight"),
        ff_norm=RMSNormSpec("rmsnorm", H, eps, p + "post_attention_layernorm.weight"),
        ff=SwiGLUSpec("swiglu", hidden=H, intermediate=I, gate=p + "mlp.gate_proj.weight",
                      up=p + "mlp.up_proj.weight", down=p + "mlp.down_proj.weight"))
    block = build_part("block", spec, env_for(dtype))
    assert sorted(n.name for n in block.tensor_needs()) == sorted(w)
    block.load(loader(w, dtype))
    T = 21
    ctx, table, n_pages = make_context([T], [0], dtype)
    kc = torch.zeros(n_pages, nKV, PAGE, d, dtype=tdt, device="cuda")
    x = r(T, H)
    stream = ResidualStream(x.cuda().clone())
    block.forward(ctx, stream, LayerCache(kc, torch.zeros_like(kc), table, PAGE, True), None)
    pending = stream.pending if stream.pending.dim() == 2 else stream.pending.sum(0)
    got = stream.resid + pending.float()
    c = dict(num_attention_heads=nH, num_key_value_heads=nKV, head_dim=d, rope_theta=1e4, rope_scaling=None,
             rms_norm_eps=eps)
    close(got, P.decoder_layer(x, torch.arange(T), w, 0, c), dtype, "prenorm block")
