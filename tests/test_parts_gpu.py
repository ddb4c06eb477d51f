"""Each part a layer is put together from, built from its description and run alone (through the
host library's part handle) against the plain implementation's function for it, at sizes other
than the tiny models'."""

import pytest
import torch

import plain_llama as P
from helpers import TOL, rel_err

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]
PAGE = 64
DEV = "cuda:0"


def part(category, spec, dtype, max_positions=512):
    from libllm_b200.parts import PartHandle
    return PartHandle(category, spec, dtype, max_positions)


class Step:
    """A step's description built by hand: sequences of ``q_lens`` new tokens behind
    ``past_lens`` cached ones, every sequence with pages of its own."""

    def __init__(self, q_lens, past_lens, vocab=100, seed=0):
        B, T = len(q_lens), sum(q_lens)
        g = torch.Generator().manual_seed(seed)
        i32 = dict(dtype=torch.int32, device=DEV)
        self.keep = dict(
            tokens=torch.randint(0, vocab, (T,), generator=g).to(**i32),
            tok_seq=torch.cat([torch.full((n,), b) for b, n in enumerate(q_lens)]).to(**i32),
            tok_pos=torch.cat([torch.arange(p, p + n) for n, p in zip(q_lens, past_lens)]).to(**i32),
            seq_start=torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0))).to(**i32),
            seq_past=torch.tensor(past_lens).to(**i32), seq_slot=torch.arange(B).to(**i32))
        self.width = max((p + n + PAGE - 1) // PAGE for n, p in zip(q_lens, past_lens))
        # pages handed out in a scattered order: sequence b's logical page j is page j * B + b
        self.table = torch.tensor([[j * B + b for j in range(self.width)] for b in range(B)]).to(**i32)
        self.n_pages = self.width * B
        self.json = dict(n_tokens=T, n_seqs=B, q_lens=list(q_lens), past_lens=list(past_lens), slots=list(range(B)),
                         max_q_len=max(q_lens), max_kv_len=max(p + n for n, p in zip(q_lens, past_lens)),
                         decode_only=all(n == 1 for n in q_lens), **{k: v.data_ptr() for k, v in self.keep.items()})


def act(t):
    return dict(ptr=t.data_ptr(), dtype=str(t.dtype).replace("torch.", ""), rows=t.shape[-2], cols=t.shape[-1])


def close(got, ref, dtype, what):
    e = rel_err(got, ref)
    assert e < TOL[dtype][0], f"{what}: rel err {e:.3e} ({dtype})"


def summed(view):
    t = view.torch().float()
    return t.sum(0) if t.dim() == 3 else t


@pytest.mark.parametrize("dtype", DTYPES)
def test_rmsnorm_part_applies_the_pending_addition(dtype):
    H, eps = 104, 3e-4
    w = {"n.weight": 1 + 0.1 * torch.randn(H)}
    norm = part("norm", dict(kind="rmsnorm", size=H, eps=eps, weight="n.weight"), dtype)
    assert norm.description["tensor_needs"] == [dict(name="n.weight", shape=[H], role="vector", optional=False)]
    norm.load(w)
    step = Step([5, 2], [0, 0])
    resid0 = torch.randn(7, H, device=DEV)
    pending = torch.randn(7, H, device=DEV)
    resid = resid0.clone()
    out = norm.forward(dict(step=step.json, hidden=H, resid=resid.data_ptr(), pending=act(pending)))
    assert out["pending"] is None                                 # applied
    assert torch.equal(resid, resid0 + pending)                   # the stream itself moves on, in 32-bit
    ref = P.rms_norm((resid0 + pending).cpu(), w["n.weight"], eps)
    close(out["out"].torch(), ref, dtype, "rmsnorm part")
    # a subset of rows (the last norm before the output matrix) leaves the stream alone
    rows = torch.tensor([6, 1], dtype=torch.int32, device=DEV)
    before = resid.clone()
    out = norm.forward(dict(step=step.json, hidden=H, resid=resid.data_ptr(), pending=None, rows=rows.data_ptr(), n_rows=2))
    assert torch.equal(resid, before)
    close(out["out"].torch(), ref[[6, 1]], dtype, "rmsnorm part, chosen rows")


def test_rope_part_holds_the_table_of_the_plain_frequencies():
    sc = dict(rope_type="llama3", factor=4.0, low_freq_factor=1.0, high_freq_factor=8.0,
              original_max_position_embeddings=128)
    rope = part("position", dict(kind="rope", head_dim=48, rotary_dim=48, theta=30000.0, scaling=sc), "float32", 300)
    rope.load({})
    table = rope.forward(dict(step=Step([1], [0]).json))["table"].torch()
    f = P.rope_frequencies(48, 30000.0, sc)
    angle = torch.arange(300, dtype=torch.float64)[:, None] * f[None, :]
    ref = torch.cat([angle.cos(), angle.sin()], 1)
    assert tuple(table.shape) == (300, 48)
    assert float((table.cpu().double() - ref).abs().max()) < 1e-6


def attention_weights(H, nH, nKV, d, seed=0):
    g = torch.Generator().manual_seed(seed)
    r = lambda *s: (torch.randn(*s, generator=g) * 0.08).to(torch.bfloat16).float()
    return {"a.q_proj.weight": r(nH * d, H), "a.k_proj.weight": r(nKV * d, H), "a.v_proj.weight": r(nKV * d, H),
            "a.o_proj.weight": r(H, nH * d)}


def attention_spec(H, nH, nKV, d, window, position="rope"):
    pos = dict(kind="rope", head_dim=d, rotary_dim=d, theta=10000.0, scaling=None) if position == "rope" else None
    return dict(kind="attention", hidden=H, n_heads=nH, n_kv_heads=nKV, head_dim=d, position=pos, window=window,
                q="a.q_proj.weight", k="a.k_proj.weight", v="a.v_proj.weight", o="a.o_proj.weight")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,nH,nKV,d,window", [(72, 6, 2, 16, None), (40, 5, 5, 32, None), (64, 2, 1, 48, 37)])
def test_attention_part_prompt_then_single_tokens(dtype, H, nH, nKV, d, window):
    """The mixer alone: a prompt in one call, then tokens one by one, against the plain
    attention over the whole sequence; two sequences of unequal lengths share the calls."""
    tdt = getattr(torch, dtype)
    w = attention_weights(H, nH, nKV, d)
    mixer = part("mixer", attention_spec(H, nH, nKV, d, window), dtype)
    mixer.load(w)
    need = mixer.description["cache"]
    assert (need["n_kv_heads"], need["k_dim"], need["v_dim"], need["window"]) == (nKV, d, d, window)
    assert need["kind"] == ("window" if window else "full")
    lens = [70, 9]
    total = [lens[0] + 3, lens[1] + 3]
    g = torch.Generator().manual_seed(5)
    xs = [torch.randn(n, H, generator=g).to(torch.bfloat16).float() for n in total]
    c = dict(num_attention_heads=nH, num_key_value_heads=nKV, head_dim=d, rope_theta=10000.0, rope_scaling=None)
    refs = [P.attention_block(x, torch.arange(x.shape[0]), w, "a.", c, window) for x in xs]
    kc = vc = None
    outs = [[], []]
    for i in range(4):
        q_lens = lens if i == 0 else [1, 1]
        past = [0, 0] if i == 0 else [lens[0] + i - 1, lens[1] + i - 1]
        step = Step(q_lens, past)
        if kc is None:
            kc = torch.zeros(step.n_pages + 8, nKV, PAGE, d, dtype=tdt, device=DEV)
            vc = torch.zeros_like(kc)
        x = torch.cat([xs[b][past[b]:past[b] + q_lens[b]] for b in range(2)]).to(tdt).to(DEV)
        out = summed(mixer.forward(dict(step=step.json, x=act(x),
                                        cache=dict(k=kc.data_ptr(), v=vc.data_ptr(), n_pages=kc.shape[0],
                                                   page_table=step.table.data_ptr(), table_width=step.width, writes=True)))["out"])
        o = 0
        for b in range(2):
            outs[b].append(out[o:o + q_lens[b]].cpu())
            o += q_lens[b]
    for b in range(2):
        close(torch.cat(outs[b]), refs[b], dtype, f"attention part, sequence {b}")


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_part_without_a_position_encoding(dtype):
    """``position: null``: queries and keys are used as they come.  The plain attention with all
    angles zero is the same thing."""
    H, nH, nKV, d = 48, 4, 2, 16
    tdt = getattr(torch, dtype)
    w = attention_weights(H, nH, nKV, d, seed=3)
    mixer = part("mixer", attention_spec(H, nH, nKV, d, None, position=None), dtype)
    mixer.load(w)
    T = 40
    x = (torch.randn(T + 2, H, generator=torch.Generator().manual_seed(8))).to(torch.bfloat16).float()
    q = P.linear(x.double(), w["a.q_proj.weight"].double()).view(T + 2, nH, d)
    k = P.linear(x.double(), w["a.k_proj.weight"].double()).view(T + 2, nKV, d)
    v = P.linear(x.double(), w["a.v_proj.weight"].double()).view(T + 2, nKV, d)
    ref = P.linear(P.attention_scores_softmax_values(q, k, v, None).reshape(T + 2, nH * d), w["a.o_proj.weight"].double())
    kc = torch.zeros(4, nKV, PAGE, d, dtype=tdt, device=DEV)
    vc = torch.zeros_like(kc)
    got = []
    for q_lens, past in (([T], [0]), ([1], [T]), ([1], [T + 1])):
        step = Step(q_lens, past)
        xin = x[past[0]:past[0] + q_lens[0]].to(tdt).to(DEV)
        got.append(summed(mixer.forward(dict(step=step.json, x=act(xin),
                                             cache=dict(k=kc.data_ptr(), v=vc.data_ptr(), n_pages=4, page_table=step.table.data_ptr(),
                                                        table_width=step.width, writes=True)))["out"]).cpu())
    close(torch.cat(got), ref, dtype, "attention without a position encoding")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T,H,I", [(1, 40, 104), (37, 72, 200)])
def test_swiglu_part(dtype, T, H, I):
    g = torch.Generator().manual_seed(1)
    r = lambda *s: (torch.randn(*s, generator=g) * 0.1).to(torch.bfloat16).float()
    w = {"m.gate_proj.weight": r(I, H), "m.up_proj.weight": r(I, H), "m.down_proj.weight": r(H, I)}
    ff = part("feed_forward", dict(kind="swiglu", hidden=H, intermediate=I, gate="m.gate_proj.weight",
                                   up="m.up_proj.weight", down="m.down_proj.weight"), dtype)
    ff.load(w)
    x = r(T, H)
    out = summed(ff.forward(dict(step=Step([T], [0]).json, x=act(x.to(getattr(torch, dtype)).to(DEV))))["out"])
    close(out, P.feed_forward(x, w, "m."), dtype, "swiglu part")


@pytest.mark.parametrize("dtype", DTYPES)
def test_prenorm_block_alone(dtype):
    """A whole layer from its description against the plain layer: the block adds nothing of
    its own to what its parts compute, and leaves the last addition pending."""
    H, nH, nKV, d, I, eps = 48, 3, 3, 16, 88, 2e-5
    tdt = getattr(torch, dtype)
    g = torch.Generator().manual_seed(2)
    r = lambda *s: (torch.randn(*s, generator=g) * 0.1).to(torch.bfloat16).float()
    p = "model.layers.0."
    w = {p + "self_attn.q_proj.weight": r(nH * d, H), p + "self_attn.k_proj.weight": r(nKV * d, H),
         p + "self_attn.v_proj.weight": r(nKV * d, H), p + "self_attn.o_proj.weight": r(H, nH * d),
         p + "mlp.gate_proj.weight": r(I, H), p + "mlp.up_proj.weight": r(I, H), p + "mlp.down_proj.weight": r(H, I),
         p + "input_layernorm.weight": 1 + r(H), p + "post_attention_layernorm.weight": 1 + r(H)}
    norm = lambda name: dict(kind="rmsnorm", size=H, eps=eps, weight=p + name)
    spec = dict(kind="prenorm", mixer_norm=norm("input_layernorm.weight"),
                mixer=dict(kind="attention", hidden=H, n_heads=nH, n_kv_heads=nKV, head_dim=d,
                           position=dict(kind="rope", head_dim=d, rotary_dim=d, theta=1e4, scaling=None),
                           q=p + "self_attn.q_proj.weight", k=p + "self_attn.k_proj.weight",
                           v=p + "self_attn.v_proj.weight", o=p + "self_attn.o_proj.weight"),
                ff_norm=norm("post_attention_layernorm.weight"),
                ff=dict(kind="swiglu", hidden=H, intermediate=I, gate=p + "mlp.gate_proj.weight",
                        up=p + "mlp.up_proj.weight", down=p + "mlp.down_proj.weight"))
    block = part("block", spec, dtype)
    assert sorted(n["name"] for n in block.description["tensor_needs"]) == sorted(w)
    block.load(w)
    T = 21
    step = Step([T], [0])
    kc = torch.zeros(step.n_pages, nKV, PAGE, d, dtype=tdt, device=DEV)
    vc = torch.zeros_like(kc)
    x = r(T, H)
    resid = x.to(DEV).clone()
    out = block.forward(dict(step=step.json, hidden=H, resid=resid.data_ptr(), pending=None,
                             cache=dict(k=kc.data_ptr(), v=vc.data_ptr(), n_pages=kc.shape[0], page_table=step.table.data_ptr(),
                                        table_width=step.width, writes=True)))
    got = resid + summed(out["pending"])
    c = dict(num_attention_heads=nH, num_key_value_heads=nKV, head_dim=d, rope_theta=1e4, rope_scaling=None,
             rms_norm_eps=eps)
    close(got, P.decoder_layer(x, torch.arange(T), w, 0, c), dtype, "prenorm block")


def test_a_part_refuses_what_it_cannot_do():
    from libllm_b200.errors import ConfigError, UnsupportedError, WeightsError
    with pytest.raises(UnsupportedError, match="head size 24"):
        part("mixer", attention_spec(48, 2, 1, 24, None), "bfloat16")
    with pytest.raises(ConfigError, match="not a multiple"):
        part("mixer", attention_spec(48, 3, 2, 16, None), "bfloat16")
    with pytest.raises(ConfigError, match="no feed_forward of kind 'gelu_mlp'.*swiglu"):
        part("feed_forward", dict(kind="gelu_mlp"), "bfloat16")
    with pytest.raises(ConfigError, match="'eps'"):
        part("norm", dict(kind="rmsnorm", size=8, weight="w"), "float32")
    ff = part("feed_forward", dict(kind="swiglu", hidden=8, intermediate=16, gate="g", up="u", down="d"), "float32")
    with pytest.raises(WeightsError) as e:
        ff.load({"g": torch.zeros(16, 8), "u": torch.zeros(8, 16), "x": torch.zeros(1)})
    assert e.value.missing == ["d"] and e.value.unexpected == ["x"] and e.value.wrong_shape[0][0] == "u"
