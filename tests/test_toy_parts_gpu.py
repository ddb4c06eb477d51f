"""Parts and an architecture that exist only in this file are registered, built and
stepped through the library's engine without a change to the library's files:

* a mixer with fixed-size state of its own per sequence (a decaying memory),
* a feed-forward that routes each token to one of several experts,
* another position encoding (angles that grow linearly with the channel),
* an order of layers that names a layer twice and lets a run read another run's cache,
* two kinds of attention (all keys, a window of them) in one model, so that the cache
  holds two groups of layers with storage of their own.

The toy parts compute with torch operators on the device (they are test doubles, not
product kernels); the plain implementation below restates the same model on the CPU in
float64 for whole sequences.  None of this is a model of the reference's or of anyone's."""
from dataclasses import dataclass

import pytest
import torch

import plain_llama as P
from helpers import check_logits
from replay import replay_batch

pytestmark = pytest.mark.gpu

H, V, D, NH, NKV, I, E, MEM = 48, 97, 16, 3, 1, 80, 3, 24
WINDOW, EPS, DECAY = 20, 1e-5, 0.8


# ------------------------------------------------------------------------- the toy parts
def register_toys():
    from libllm_b200.config import ModelConfig, register_architecture
    from libllm_b200.parts.base import FeedForward, Mixer, PositionEncoding, StateNeed
    from libllm_b200.parts.registry import register_part
    from libllm_b200.parts.spec import (AttentionSpec, BlockSpec, ModelSpec, PartSpec, RMSNormSpec, RopeSpec,
                                        ScheduleEntry, SwiGLUSpec)
    from libllm_b200.weights.state_map import TensorNeed

    @dataclass(frozen=True)
    class MemorySpec(PartSpec):
        hidden: int = 0
        size: int = 0
        decay: float = 0.5
        w_in: str = ""
        w_out: str = ""

    @dataclass(frozen=True)
    class RoutedSpec(PartSpec):
        hidden: int = 0
        intermediate: int = 0
        experts: int = 0
        prefix: str = ""

    @dataclass(frozen=True)
    class LinearAngleSpec(PartSpec):
        head_dim: int = 0
        step: float = 0.01

    class DecayingMemory(Mixer):
        """s_t = decay * s_(t-1) + W_in x_t;  y_t = W_out s_t.  The state s is kept per
        sequence between steps; single-token steps touch it through device indices only,
        so they can be captured in a graph."""

        def tensor_needs(self):
            s = self.spec
            return [TensorNeed(s.w_in, (s.size, s.hidden)), TensorNeed(s.w_out, (s.hidden, s.size))]

        def load(self, fetch):
            needs = self.tensor_needs()
            self.w_in, self.w_out = fetch(needs[0]).float(), fetch(needs[1]).float()

        def state_need(self):
            return {"s": StateNeed((self.spec.size,), torch.float32)}

        def forward(self, ctx, x, cache, state):
            assert cache is None
            u = x.float() @ self.w_in.t()
            store = state["s"]
            slots = ctx.seq_slot[:ctx.n_seqs].long()
            if ctx.decode_only:
                s = self.spec.decay * store[slots] + u
                store.index_copy_(0, slots, s)
                return s @ self.w_out.t()
            out = torch.empty_like(u)
            o = 0
            for b, n in enumerate(ctx.q_lens):
                s = store[ctx.slots[b]].clone()
                for t in range(n):
                    s = self.spec.decay * s + u[o + t]
                    out[o + t] = s
                store[ctx.slots[b]] = s
                o += n
            return out @ self.w_out.t()

    class RoutedExperts(FeedForward):
        """Router logits in 32-bit, the most probable expert alone, its SwiGLU scaled by
        the router's probability for it."""

        def tensor_needs(self):
            s, p = self.spec, self.spec.prefix
            needs = [TensorNeed(p + "router.weight", (s.experts, s.hidden), role="vector")]
            for e in range(s.experts):
                needs += [TensorNeed(f"{p}experts.{e}.gate_proj.weight", (s.intermediate, s.hidden)),
                          TensorNeed(f"{p}experts.{e}.up_proj.weight", (s.intermediate, s.hidden)),
                          TensorNeed(f"{p}experts.{e}.down_proj.weight", (s.hidden, s.intermediate))]
            return needs

        def load(self, fetch):
            needs = self.tensor_needs()
            self.router = fetch(needs[0]).float()
            w = [fetch(n).float() for n in needs[1:]]
            self.gate, self.up, self.down = (torch.stack(w[i::3]) for i in range(3))

        def forward(self, ctx, x):
            xf = x.float()
            prob = torch.softmax(xf @ self.router.t(), dim=-1)
            top, idx = prob.max(dim=-1)
            g = torch.einsum("th,tih->ti", xf, self.gate[idx])
            u = torch.einsum("th,tih->ti", xf, self.up[idx])
            m = (g / (1 + torch.exp(-g)) * u).to(x.dtype).float()      # rounded where the engine stores it
            return torch.einsum("ti,thi->th", m, self.down[idx]) * top[:, None]

    class LinearAngles(PositionEncoding):
        """Rotation by angle p * step * (i + 1) for channel pair i: the same table
        interface as the rotary part ([positions, d]: cosines, then sines)."""

        def __init__(self, spec, env):
            super().__init__(spec, env)
            self.table = None

        def load(self, fetch):
            d = self.spec.head_dim
            f = self.spec.step * torch.arange(1, d // 2 + 1, dtype=torch.float64, device=self.env.device)
            a = torch.arange(self.env.max_positions, dtype=torch.float64, device=self.env.device)[:, None] * f
            self.table = torch.cat([a.cos(), a.sin()], 1).float().contiguous()

    for cat, kind, cls in (("mixer", "toy_memory", DecayingMemory), ("feed_forward", "toy_routed", RoutedExperts),
                           ("position", "toy_linear_angles", LinearAngles)):
        register_part(cat, kind, cls, replace=True)

    @dataclass(frozen=True)
    class ToyConfig(ModelConfig):
        vocab_size: int = 0

    def parse(data):
        return ToyConfig(model_type=data["model_type"], vocab_size=int(data["vocab_size"]))

    def describe(c):
        def attn(i, position, window):
            p = f"layers.{i}.attn."
            return AttentionSpec("attention", hidden=H, n_heads=NH, n_kv_heads=NKV, head_dim=D, position=position,
                                 window=window, q=p + "q_proj.weight", k=p + "k_proj.weight",
                                 v=p + "v_proj.weight", o=p + "o_proj.weight")

        def norm(name):
            return RMSNormSpec("rmsnorm", H, EPS, name)

        def swiglu(i):
            p = f"layers.{i}.mlp."
            return SwiGLUSpec("swiglu", hidden=H, intermediate=I, gate=p + "gate_proj.weight",
                              up=p + "up_proj.weight", down=p + "down_proj.weight")
        layers = (
            BlockSpec("prenorm", norm("layers.0.n1.weight"),
                      attn(0, RopeSpec("rope", head_dim=D, rotary_dim=D, theta=1e4, scaling=None), None),
                      norm("layers.0.n2.weight"), swiglu(0)),
            BlockSpec("prenorm", norm("layers.1.n1.weight"),
                      MemorySpec("toy_memory", hidden=H, size=MEM, decay=DECAY, w_in="layers.1.mem.in.weight",
                                 w_out="layers.1.mem.out.weight"),
                      norm("layers.1.n2.weight"),
                      RoutedSpec("toy_routed", hidden=H, intermediate=I, experts=E, prefix="layers.1.moe.")),
            BlockSpec("prenorm", norm("layers.2.n1.weight"),
                      attn(2, LinearAngleSpec("toy_linear_angles", head_dim=D, step=0.01), WINDOW),
                      norm("layers.2.n2.weight"), swiglu(2)),
        )
        schedule = (ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(2), ScheduleEntry(1),
                    ScheduleEntry(0, cache_from=0))
        return ModelSpec(vocab_size=c.vocab_size, hidden=H, embedding="embed.weight", layers=layers,
                         schedule=schedule, final_norm=norm("norm.weight"), head="head.weight",
                         max_positions=512, stop_tokens=(), name="toy_hybrid")

    register_architecture("toy_hybrid", parse, describe, replace=True)


# ------------------------------------------------------------------------- the plain form
def plain_attention(x, w, prefix, freqs, window, kv=None):
    T = x.shape[0]
    pos = torch.arange(T)
    q = P.rope_rotate(P.linear(x, w[prefix + "q_proj.weight"]).view(T, NH, D), pos, freqs)
    if kv is None:
        k = P.rope_rotate(P.linear(x, w[prefix + "k_proj.weight"]).view(T, NKV, D), pos, freqs)
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


def plain_forward(w, ids):
    x = P.embedding(w["embed.weight"], ids)
    rope = P.rope_frequencies(D, 1e4, None)
    lin = 0.01 * torch.arange(1, D // 2 + 1, dtype=torch.float64)
    n = lambda x, name: P.rms_norm(x, w[name], EPS)
    # entry 0: layer 0 (keeps its keys and values)
    a, kv0 = plain_attention(n(x, "layers.0.n1.weight"), w, "layers.0.attn.", rope, None)
    x = x + a
    x = x + P.feed_forward(n(x, "layers.0.n2.weight"), w, "layers.0.mlp.")
    for entry in (1, 2, 3):
        if entry == 2:
            a, _ = plain_attention(n(x, "layers.2.n1.weight"), w, "layers.2.attn.", lin, WINDOW)
            x = x + a
            x = x + P.feed_forward(n(x, "layers.2.n2.weight"), w, "layers.2.mlp.")
        else:                     # layer 1, twice; each run's memory starts at zero
            x = x + plain_memory(n(x, "layers.1.n1.weight"), w)
            x = x + plain_routed(n(x, "layers.1.n2.weight"), w)
    # entry 4: layer 0 again, its queries over the keys and values that entry 0 kept
    a, _ = plain_attention(n(x, "layers.0.n1.weight"), w, "layers.0.attn.", rope, None, kv=kv0)
    x = x + a
    x = x + P.feed_forward(n(x, "layers.0.n2.weight"), w, "layers.0.mlp.")
    return P.linear(n(x, "norm.weight"), w["head.weight"])


# ------------------------------------------------------------------------- the tests
_built = {}


def toy_engine(dtype, max_tokens=2048):
    if dtype not in _built:
        register_toys()
        from libllm_b200.engine import Engine, Model
        from libllm_b200.weights.random_model import random_tensors
        cfg = dict(model_type="toy_hybrid", vocab_size=V)
        tensors = random_tensors(cfg, seed=4, dtype=torch.bfloat16)
        # Routing must not hinge on rounding: the token table marks each id's expert (id % E)
        # in one of its first E channels, far above everything else in the row, and the
        # router reads just these channels.  The chosen expert's probability stays near 0.8.
        emb = tensors["embed.weight"]
        emb[:, :E] = 0
        emb[torch.arange(V), torch.arange(V) % E] = 4.0
        router = torch.zeros(E, H)
        router[torch.arange(E), torch.arange(E)] = 0.3
        tensors["layers.1.moe.router.weight"] = router
        from libllm_b200.config import architecture_for
        config = architecture_for("toy_hybrid").parse(cfg)
        model = Model.from_tensors(config, tensors, dtype=dtype, device="cuda:0")
        _built[dtype] = (Engine(model, max_tokens=max_tokens), {k: v.double() for k, v in tensors.items()})
    return _built[dtype]


def toks(n, seed):
    return torch.randint(0, V, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_model_is_described_by_data(dtype):
    engine, _ = toy_engine(dtype)
    cache = engine.cache
    kinds = sorted((g.need.kind, g.need.window, len(g.runs)) for g in cache.groups)
    assert kinds == [("full", None, 1), ("window", WINDOW, 1)]      # entry 4 owns no storage
    assert cache.run_group[1] is None and cache.run_group[4] is None
    assert [sorted(s) for s in cache.state] == [[], ["s"], [], ["s"], []]
    assert cache.state[1]["s"].data_ptr() != cache.state[3]["s"].data_ptr()   # a state per run, not per layer


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_model_whole_then_token_by_token_in_unequal_batches(dtype):
    engine, w = toy_engine(dtype)
    for b in range(2):                         # the second batch gets the first one's slots and pages
        reqs = [(f"{b}a", toks(75, 10 * b), 40), (f"{b}b", toks(9, 10 * b + 1), 3), (f"{b}c", toks(50, 10 * b + 2), 50)]
        got = replay_batch(engine, reqs)
        for rid, t, _ in reqs:
            check_logits(got[rid], plain_forward(w, t), dtype, f"toy {rid}")
    assert all(g.pool.in_use == 0 for g in engine.cache.groups)


def test_window_group_gives_pages_back_while_the_full_group_keeps_them():
    from libllm_b200.engine import StepItem
    engine, _ = toy_engine("float32")
    s = engine.open_sequence()
    engine.step([StepItem(s, toks(200, 3), [])])
    used = {g.need.kind: g.pool.in_use for g in engine.cache.groups}
    assert used["full"] == 4 and used["window"] == 2          # 200 tokens: 4 pages; keys 181..199 lie in two
    engine.close_sequence(s)
    engine.cache.check()
