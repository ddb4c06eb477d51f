"""Parts and architectures that exist only in this file are registered, built and stepped
through the library's engine without a change to the library's files:

* a mixer with fixed-size state of its own per sequence (a decaying memory),
* a mixer that keeps keys and values of different widths in the cache,
* a feed-forward that routes each token to one of several experts,
* another position encoding (angles that grow linearly with the channel),
* an attention layer without any position encoding,
* an order of layers that names a layer twice and lets a run read another run's cache,
* two kinds of attention (all keys, a window of them) in one model, so that the cache
  holds groups of layers with storage of their own,
* a token table that is scaled and logits that are scaled and capped.

The toy parts are Python classes registered through the library's plug-in interface
(include/llm_plugin.h); they compute with torch operators on the step's stream (they are test
doubles, not product kernels).  The plain implementations below restate the same models on the
CPU in float64 for whole sequences.  None of this is a model of the reference's or of anyone's."""
import math

import pytest
import torch

import plain_llama as P
from helpers import check_logits
from replay import replay_batch

pytestmark = pytest.mark.gpu

H, V, D, NH, NKV, I, E, MEM = 48, 97, 16, 3, 1, 80, 3, 24
DK, DV = 8, 24
WINDOW, EPS, DECAY = 20, 1e-5, 0.8
EMB_SCALE, LOGIT_SCALE, SOFTCAP = 1.5, 0.5, 6.0


# ------------------------------------------------------------------------- the toy parts
class DecayingMemory:
    """s_t = decay * s_(t-1) + W_in x_t;  y_t = W_out s_t.  The state s is kept per sequence
    between steps."""

    def __init__(self, spec, env):
        self.spec, self.w = spec, {}

    def tensor_needs(self):
        s = self.spec
        return [dict(name=s["w_in"], shape=[s["size"], s["hidden"]]), dict(name=s["w_out"], shape=[s["hidden"], s["size"]])]

    def load_tensor(self, name, tensor):
        self.w[name] = tensor.torch().float()

    def needs(self):
        return dict(cache=None, state=[dict(name="s", shape=[self.spec["size"]], dtype="float32")])

    def forward(self, step, x, cache, state, out):
        assert cache is None
        with step.torch_stream():
            w_in, w_out = self.w[self.spec["w_in"]], self.w[self.spec["w_out"]]
            u = x.torch().float() @ w_in.t()
            store = state["s"].torch()
            y = torch.empty_like(u)
            o = 0
            for b, n in enumerate(step.q_lens):
                s = store[step.slots[b]].clone()
                for t in range(n):
                    s = self.spec["decay"] * s + u[o + t]
                    y[o + t] = s
                store[step.slots[b]] = s
                o += n
            out.torch().copy_(y @ w_out.t())


class WideValueAttention:
    """One head whose keys are DK wide and whose values are DV wide, kept in the paged cache
    ([pages, 1, page, DK] and [pages, 1, page, DV]); no position encoding."""

    def __init__(self, spec, env):
        self.spec, self.w = spec, {}

    def tensor_needs(self):
        p, s = self.spec["prefix"], self.spec
        return [dict(name=p + "q.weight", shape=[s["dk"], s["hidden"]]), dict(name=p + "k.weight", shape=[s["dk"], s["hidden"]]),
                dict(name=p + "v.weight", shape=[s["dv"], s["hidden"]]), dict(name=p + "o.weight", shape=[s["hidden"], s["dv"]])]

    def load_tensor(self, name, tensor):
        self.w[name[len(self.spec["prefix"]):]] = tensor.torch().float()

    def needs(self):
        return dict(cache=dict(kind="full", n_kv_heads=1, k_dim=self.spec["dk"], v_dim=self.spec["dv"]), state=[])

    def forward(self, step, x, cache, state, out):
        assert cache.k_dim == self.spec["dk"] and cache.v_dim == self.spec["dv"] and cache.writes
        with step.torch_stream():
            xf = x.torch().float()
            q, k, v = xf @ self.w["q.weight"].t(), xf @ self.w["k.weight"].t(), xf @ self.w["v.weight"].t()
            kc, vc, table = cache.k.torch(), cache.v.torch(), cache.page_table.torch().long()
            P_ = cache.page_size
            y = torch.empty(xf.shape[0], self.spec["dv"], device=xf.device)
            o = 0
            for b, (n, past) in enumerate(zip(step.q_lens, step.past_lens)):
                pos = torch.arange(past, past + n, device=xf.device)
                pages = table[b, pos // P_]
                kc[pages, 0, pos % P_] = k[o:o + n].to(kc.dtype)
                vc[pages, 0, pos % P_] = v[o:o + n].to(vc.dtype)
                allpos = torch.arange(0, past + n, device=xf.device)
                K = kc[table[b, allpos // P_], 0, allpos % P_].float()
                Vv = vc[table[b, allpos // P_], 0, allpos % P_].float()
                s = (q[o:o + n] @ K.t()) / math.sqrt(self.spec["dk"])
                s = s.masked_fill(allpos[None, :] > pos[:, None], float("-inf"))
                y[o:o + n] = torch.softmax(s, dim=-1) @ Vv
                o += n
            out.torch().copy_(y @ self.w["o.weight"].t())


class RoutedExperts:
    """Router logits in 32-bit, the most probable expert alone, its SwiGLU scaled by the router's
    probability for it."""

    def __init__(self, spec, env):
        self.spec, self.env, self.w = spec, env, {}

    def tensor_needs(self):
        s, p = self.spec, self.spec["prefix"]
        needs = [dict(name=p + "router.weight", shape=[s["experts"], s["hidden"]], role="vector")]
        for e in range(s["experts"]):
            needs += [dict(name=f"{p}experts.{e}.gate_proj.weight", shape=[s["intermediate"], s["hidden"]]),
                      dict(name=f"{p}experts.{e}.up_proj.weight", shape=[s["intermediate"], s["hidden"]]),
                      dict(name=f"{p}experts.{e}.down_proj.weight", shape=[s["hidden"], s["intermediate"]])]
        return needs

    def load_tensor(self, name, tensor):
        self.w[name[len(self.spec["prefix"]):]] = tensor.torch().float()

    def forward(self, step, x, out):
        with step.torch_stream():
            n = self.spec["experts"]
            gate = torch.stack([self.w[f"experts.{e}.gate_proj.weight"] for e in range(n)])
            up = torch.stack([self.w[f"experts.{e}.up_proj.weight"] for e in range(n)])
            down = torch.stack([self.w[f"experts.{e}.down_proj.weight"] for e in range(n)])
            xf = x.torch().float()
            prob = torch.softmax(xf @ self.w["router.weight"].t(), dim=-1)
            top, idx = prob.max(dim=-1)
            g = torch.einsum("th,tih->ti", xf, gate[idx])
            u = torch.einsum("th,tih->ti", xf, up[idx])
            m = (g / (1 + torch.exp(-g)) * u).to(x.torch().dtype).float()      # rounded where the engine stores it
            out.torch().copy_(torch.einsum("ti,thi->th", m, down[idx]) * top[:, None])


class LinearAngles:
    """Rotation by angle p * step * (i + 1) for channel pair i: a table of its own angles
    ([positions, d]: cosines, then sines) for the library's rotation kernels."""

    def __init__(self, spec, env):
        self.spec, self.env, self._table = spec, env, None

    def table(self):
        if self._table is None:
            d = self.spec["head_dim"]
            f = self.spec["step"] * torch.arange(1, d // 2 + 1, dtype=torch.float64, device="cuda")
            a = torch.arange(self.env["max_positions"], dtype=torch.float64, device="cuda")[:, None] * f
            self._table = torch.cat([a.cos(), a.sin()], 1).float().contiguous()
            torch.cuda.synchronize()
        return self._table.data_ptr(), self._table.shape[0], self._table.shape[1]


def norm(name):
    return dict(kind="rmsnorm", size=H, eps=EPS, weight=name)


def attn(i, position, window):
    p = f"layers.{i}.attn."
    return dict(kind="attention", hidden=H, n_heads=NH, n_kv_heads=NKV, head_dim=D, position=position, window=window,
                q=p + "q_proj.weight", k=p + "k_proj.weight", v=p + "v_proj.weight", o=p + "o_proj.weight")


def swiglu(i):
    p = f"layers.{i}.mlp."
    return dict(kind="swiglu", hidden=H, intermediate=I, gate=p + "gate_proj.weight", up=p + "up_proj.weight",
                down=p + "down_proj.weight")


def block(i, mixer, ff):
    return dict(kind="prenorm", mixer_norm=norm(f"layers.{i}.n1.weight"), mixer=mixer, ff_norm=norm(f"layers.{i}.n2.weight"), ff=ff)


ROPE = dict(kind="rope", head_dim=D, rotary_dim=D, theta=1e4, scaling=None)
LINEAR = dict(kind="toy_linear_angles", head_dim=D, step=0.01)


def describe_hybrid(c):
    layers = [block(0, attn(0, ROPE, None), swiglu(0)),
              block(1, dict(kind="toy_memory", hidden=H, size=MEM, decay=DECAY, w_in="layers.1.mem.in.weight",
                            w_out="layers.1.mem.out.weight"),
                    dict(kind="toy_routed", hidden=H, intermediate=I, experts=E, prefix="layers.1.moe.")),
              block(2, attn(2, LINEAR, WINDOW), swiglu(2)),
              block(3, dict(kind="toy_wide_value", hidden=H, dk=DK, dv=DV, prefix="layers.3.wide."), swiglu(3))]
    schedule = [0, 1, 2, 1, 3, dict(layer=0, cache_from=0)]
    return dict(name="toy_hybrid", vocab_size=c["vocab_size"], hidden=H, embedding="embed.weight", layers=layers,
                schedule=schedule, final_norm=norm("norm.weight"), head="head.weight", max_positions=512, stop_tokens=[])


def describe_attn(c):
    layers = [block(0, attn(0, ROPE, None), swiglu(0)), block(1, attn(1, None, WINDOW), swiglu(1)),
              block(2, attn(2, LINEAR, None), swiglu(2))]
    schedule = [0, 1, 2, 1, dict(layer=0, cache_from=0)]
    return dict(name="toy_attn", vocab_size=c["vocab_size"], hidden=H, embedding="embed.weight", layers=layers,
                schedule=schedule, final_norm=norm("norm.weight"), head=None, max_positions=512, stop_tokens=[5],
                embedding_scale=EMB_SCALE, logit_scale=LOGIT_SCALE, logit_softcap=SOFTCAP,
                ignore_tensors=["extra.*"])


def register_toys():
    from libllm_b200.config import register_architecture
    from libllm_b200.parts import register_part
    for cat, kind, cls in (("mixer", "toy_memory", DecayingMemory), ("mixer", "toy_wide_value", WideValueAttention),
                           ("feed_forward", "toy_routed", RoutedExperts), ("position", "toy_linear_angles", LinearAngles)):
        register_part(cat, kind, cls, replace=True)

    def parse(data):
        return dict(model_type=data["model_type"], vocab_size=int(data["vocab_size"]))

    register_architecture("toy_hybrid", parse, describe_hybrid, replace=True)
    register_architecture("toy_attn", parse, describe_attn, replace=True)


# ------------------------------------------------------------------------- the plain form
def plain_attention(x, w, prefix, freqs, window, kv=None):
    T = x.shape[0]
    pos = torch.arange(T)
    rot = (lambda t: P.rope_rotate(t, pos, freqs)) if freqs is not None else (lambda t: t)
    q = rot(P.linear(x, w[prefix + "q_proj.weight"]).view(T, NH, D))
    if kv is None:
        k = rot(P.linear(x, w[prefix + "k_proj.weight"]).view(T, NKV, D))
        v = P.linear(x, w[prefix + "v_proj.weight"]).view(T, NKV, D)
        kv = (k, v)
    o = P.attention_scores_softmax_values(q, kv[0], kv[1], window)
    return P.linear(o.reshape(T, NH * D), w[prefix + "o_proj.weight"]), kv


def plain_memory(x, w):
    u = P.linear(x, w["layers.1.mem.in.weight"])
    s = torch.zeros(MEM, dtype=torch.float64)
    out = []
    for t in range(x.shape[0]):
        s = DECAY * s + u[t]
        out.append(s)
    return P.linear(torch.stack(out), w["layers.1.mem.out.weight"])


def plain_routed(x, w):
    prob = torch.softmax(P.linear(x, w["layers.1.moe.router.weight"]), dim=-1)
    out = torch.zeros(x.shape[0], H, dtype=torch.float64)
    for t in range(x.shape[0]):
        e = int(prob[t].argmax())
        out[t] = P.feed_forward(x[t:t + 1], w, f"layers.1.moe.experts.{e}.")[0] * prob[t, e]
    return out


def plain_wide(x, w):
    p = "layers.3.wide."
    q, k, v = (P.linear(x, w[p + n + ".weight"]) for n in "qkv")
    T = x.shape[0]
    s = (q @ k.t()) / math.sqrt(DK)
    s = s.masked_fill(torch.arange(T)[None, :] > torch.arange(T)[:, None], float("-inf"))
    return P.linear(torch.softmax(s, dim=-1) @ v, w[p + "o.weight"])


LIN_FREQS = 0.01 * torch.arange(1, D // 2 + 1, dtype=torch.float64)


def plain_hybrid(w, ids):
    x = P.embedding(w["embed.weight"], ids)
    rope = P.rope_frequencies(D, 1e4, None)
    n = lambda x, name: P.rms_norm(x, w[name], EPS)
    a, kv0 = plain_attention(n(x, "layers.0.n1.weight"), w, "layers.0.attn.", rope, None)     # entry 0 keeps its keys and values
    x = x + a
    x = x + P.feed_forward(n(x, "layers.0.n2.weight"), w, "layers.0.mlp.")
    for entry in (1, 2, 3, 4):
        if entry == 2:
            a, _ = plain_attention(n(x, "layers.2.n1.weight"), w, "layers.2.attn.", LIN_FREQS, WINDOW)
            x = x + a
            x = x + P.feed_forward(n(x, "layers.2.n2.weight"), w, "layers.2.mlp.")
        elif entry == 4:
            x = x + plain_wide(n(x, "layers.3.n1.weight"), w)
            x = x + P.feed_forward(n(x, "layers.3.n2.weight"), w, "layers.3.mlp.")
        else:                     # layer 1, twice; each run's memory starts at zero
            x = x + plain_memory(n(x, "layers.1.n1.weight"), w)
            x = x + plain_routed(n(x, "layers.1.n2.weight"), w)
    # the last entry: layer 0 again, its queries over the keys and values that entry 0 kept
    a, _ = plain_attention(n(x, "layers.0.n1.weight"), w, "layers.0.attn.", rope, None, kv=kv0)
    x = x + a
    x = x + P.feed_forward(n(x, "layers.0.n2.weight"), w, "layers.0.mlp.")
    return P.linear(n(x, "norm.weight"), w["head.weight"])


def plain_attn_model(w, ids):
    x = P.embedding(w["embed.weight"], ids) * EMB_SCALE
    rope = P.rope_frequencies(D, 1e4, None)
    n = lambda x, name: P.rms_norm(x, w[name], EPS)

    def layer(x, i, freqs, window, kv=None):
        a, kv = plain_attention(n(x, f"layers.{i}.n1.weight"), w, f"layers.{i}.attn.", freqs, window, kv)
        x = x + a
        return x + P.feed_forward(n(x, f"layers.{i}.n2.weight"), w, f"layers.{i}.mlp."), kv

    x, kv0 = layer(x, 0, rope, None)
    x, _ = layer(x, 1, None, WINDOW)
    x, _ = layer(x, 2, LIN_FREQS, None)
    x, _ = layer(x, 1, None, WINDOW)               # the same weights, a cache of its own
    x, _ = layer(x, 0, rope, None, kv0)
    logits = P.linear(n(x, "norm.weight"), w["embed.weight"]) * LOGIT_SCALE
    return SOFTCAP * torch.tanh(logits / SOFTCAP)


# ------------------------------------------------------------------------- the tests
_built = {}


def random_tensors(cfg, seed):
    from libllm_b200.weights import tensor_needs_of
    g = torch.Generator().manual_seed(seed)
    out = {}
    for need in tensor_needs_of(cfg):
        if need["role"] == "vector":
            t = 1 + 0.2 * (torch.rand(need["shape"], generator=g) - 0.5)
        else:
            t = 0.05 * torch.randn(need["shape"], generator=g)
        out[need["name"]] = t.to(torch.bfloat16)
    return out


def toy_engine(which, dtype, max_tokens=2048):
    key = (which, dtype)
    if key not in _built:
        register_toys()
        from libllm_b200.engine import Engine
        cfg = dict(model_type=which, vocab_size=V)
        tensors = random_tensors(cfg, seed=4)
        if which == "toy_hybrid":
            # Routing must not hinge on rounding: the token table marks each id's expert (id % E)
            # in one of its first E channels, far above everything else in the row, and the
            # router reads just these channels.  The chosen expert's probability stays near 0.8.
            emb = tensors["embed.weight"]
            emb[:, :E] = 0
            emb[torch.arange(V), torch.arange(V) % E] = 4.0
            router = torch.zeros(E, H)
            router[torch.arange(E), torch.arange(E)] = 0.3
            tensors["layers.1.moe.router.weight"] = router
        else:
            tensors["extra.unused"] = torch.zeros(3)          # covered by the description's ignore list
        engine = Engine.from_tensors(cfg, tensors, dtype=dtype, max_tokens=max_tokens)
        _built[key] = (engine, {k: v.double() for k, v in tensors.items()})
    return _built[key]


def toks(n, seed):
    return torch.randint(0, V, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_model_is_described_by_data(dtype):
    engine, _ = toy_engine("toy_hybrid", dtype)
    info = engine.cache_info()
    kinds = sorted((g["kind"], g["window"], g["k_dim"], g["v_dim"], len(g["runs"])) for g in info["groups"])
    assert kinds == [("full", None, DK, DV, 1), ("full", None, D, D, 1), ("window", WINDOW, D, D, 1)]
    assert info["run_group"][1] is None and info["run_group"][3] is None and info["run_group"][5] is None   # entry 5 owns no storage
    assert [sorted(s) for s in info["state"]] == [[], ["s"], [], ["s"], [], []]
    assert info["state"][1]["s"]["address"] != info["state"][3]["s"]["address"]       # a state per run, not per layer
    assert not engine.info()["use_graphs"]          # the Python parts read the step's host arrays
    attn_engine, _ = toy_engine("toy_attn", dtype)
    assert attn_engine.info()["use_graphs"]
    assert attn_engine.info()["ignored_tensors"] == ["extra.unused"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which,plain_forward", [("toy_hybrid", plain_hybrid), ("toy_attn", plain_attn_model)])
def test_toy_model_whole_then_token_by_token_in_unequal_batches(which, plain_forward, dtype):
    engine, w = toy_engine(which, dtype)
    for b in range(2):                         # the second batch gets the first one's slots and pages
        reqs = [(f"{b}a", toks(75, 10 * b), 40), (f"{b}b", toks(9, 10 * b + 1), 3), (f"{b}c", toks(50, 10 * b + 2), 50)]
        got = replay_batch(engine, reqs)
        for rid, t, _ in reqs:
            check_logits(got[rid], plain_forward(w, t), dtype, f"{which} {rid}")
    assert all(n == 0 for n in engine.pages_in_use())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_run_that_reads_another_runs_cache_over_hundreds_of_graph_steps(dtype):
    """The schedule's last entry attends over the keys and values that its first entry wrote a few
    launches earlier in the same step.  Three hundred single-token steps (captured graphs, the
    window group giving pages back on the way) against the plain model."""
    engine, w = toy_engine("toy_attn", dtype)
    long_, short = toks(330, 31), toks(140, 32)
    got = replay_batch(engine, [("long", long_, 30), ("short", short, 3)])
    check_logits(got["long"], plain_attn_model(w, long_), dtype, "long")
    check_logits(got["short"], plain_attn_model(w, short), dtype, "short")
    assert engine.info()["graph_replays"] > 250


def test_window_group_gives_pages_back_while_the_full_group_keeps_them():
    from libllm_b200.engine import StepItem
    engine, _ = toy_engine("toy_hybrid", "float32")
    s = engine.open_sequence()
    engine.step([StepItem(s, toks(200, 3), [])])
    used = {(g["kind"], g["k_dim"]): g["pages_in_use"] for g in engine.cache_info()["groups"]}
    assert used[("full", D)] == 4 and used[("full", DK)] == 4 and used[("window", D)] == 2   # keys 181..199 lie in two pages
    engine.close_sequence(s)
    engine.cache_check()


def test_generation_stops_at_the_toy_models_own_stop_token():
    """The description's stop tokens are the generation loop's default."""
    engine, w = toy_engine("toy_attn", "float32")
    prompt = toks(12, 77)
    ids, want = list(prompt), []
    for _ in range(20):
        t = int(plain_attn_model(w, ids)[-1].argmax())
        if t == 5:
            break
        want.append(t)
        ids.append(t)
    from libllm_b200.engine import GREEDY
    assert engine.generate([prompt], 20, GREEDY)[0] == want


def test_errors_of_a_plugin_reach_the_caller():
    from libllm_b200.config import register_architecture
    from libllm_b200.engine import Engine
    from libllm_b200.errors import ConfigError, LlmError
    from libllm_b200.parts import register_part
    register_toys()

    class Broken:
        def __init__(self, spec, env):
            raise ValueError("this part cannot be built")

    register_part("feed_forward", "toy_broken", Broken, replace=True)
    register_architecture("toy_broken_arch", lambda d: dict(model_type=d["model_type"], vocab_size=7),
                          lambda c: dict(describe_attn(c), layers=[block(0, attn(0, ROPE, None), dict(kind="toy_broken"))],
                                         schedule=[0]), replace=True)
    with pytest.raises(ConfigError, match="this part cannot be built"):
        Engine.from_tensors(dict(model_type="toy_broken_arch", vocab_size=7), {}, dtype="float32")
    with pytest.raises(ConfigError, match="registered already"):
        register_part("mixer", "toy_memory", DecayingMemory)
    with pytest.raises(LlmError, match="mixer, a feed_forward or a position"):
        register_part("norm", "toy_norm", DecayingMemory)
