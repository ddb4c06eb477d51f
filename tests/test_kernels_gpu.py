"""Each kernel alone against its plain reference, at sizes other than the engine's."""
import math

import pytest
import torch

import plain_llama as P

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
TOL = {"float32": 2e-6, "bfloat16": 1e-2}


def close(got, ref, dtype, scale=None):
    ref = ref.to(torch.float64)
    err = float((got.detach().to(torch.float64).cpu() - ref.cpu()).abs().max())
    bound = TOL[dtype] * (scale if scale is not None else float(ref.abs().max()) + 1e-30)
    assert err <= bound, f"max abs err {err:.3e} > {bound:.3e}"


def rnd(shape, dtype, seed, std=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * std).to(DT[dtype]).to(DEV)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_embedding(dtype):
    from libllm_b200.csrc import ops
    table = rnd((1000, 200), dtype, 1)
    ids = torch.tensor([0, 999, 5, 5, 321], dtype=torch.int32, device=DEV)
    out = torch.empty((5, 200), dtype=torch.float32, device=DEV)
    ops.embedding(table, ids, out)
    assert torch.equal(out.cpu(), P.embedding(table.cpu(), ids.tolist()).float())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("hidden,parts", [(200, 0), (200, 1), (72, 3), (13000, 2)])
def test_add_rmsnorm(dtype, hidden, parts):
    from libllm_b200.csrc import ops
    T = 7
    resid = rnd((T, hidden), "float32", 2)
    delta = rnd((parts, T, hidden), dtype, 3) if parts else None
    w = rnd((hidden,), "float32", 4) * 0.1 + 1
    out = torch.empty((T, hidden), dtype=DT[dtype], device=DEV)
    want = resid.double().cpu() + (delta.double().cpu().sum(0) if parts else 0)
    r2 = resid.clone()
    ops.add_rmsnorm(r2, delta, w, 1e-5, out)
    close(r2, want, "float32")
    close(out, P.rms_norm(want, w.cpu(), 1e-5), dtype)
    # a subset of rows, residual left alone
    rows = torch.tensor([6, 0, 3], dtype=torch.int32, device=DEV)
    r3 = resid.clone()
    out3 = torch.empty((3, hidden), dtype=DT[dtype], device=DEV)
    ops.add_rmsnorm(r3, delta, w, 1e-5, out3, rows)
    assert torch.equal(r3, resid)
    close(out3, P.rms_norm(want[[6, 0, 3]], w.cpu(), 1e-5), dtype)
    # add only
    r4 = resid.clone()
    ops.add_rmsnorm(r4, delta, None, 0.0, None)
    close(r4, want, "float32")


@pytest.mark.parametrize("dtype,in_dtype", [("float32", "float32"), ("bfloat16", "bfloat16"), ("bfloat16", "float32")])
@pytest.mark.parametrize("inter", [173, 176])        # the general kernel, and four values per thread
def test_swiglu(dtype, in_dtype, inter):
    from libllm_b200.csrc import ops
    gu = rnd((9, 2 * inter), in_dtype, 5, 2.0)
    gu[0, 0] = -30.0
    gu[0, 1] = 30.0
    out = torch.empty((9, inter), dtype=DT[dtype], device=DEV)
    ops.swiglu(gu, out)
    close(out, P.swiglu(gu[:, :inter].cpu(), gu[:, inter:].cpu()), dtype)


@pytest.mark.parametrize("dtype,out_dtype", [("float32", "float32"), ("bfloat16", "bfloat16"), ("bfloat16", "float32")])
@pytest.mark.parametrize("M,N,K", [(1, 1, 1), (5, 7, 3), (513, 2, 513), (70, 130, 1000), (64, 64, 16)])
def test_gemm_plain(dtype, out_dtype, M, N, K):
    from libllm_b200.csrc import ops
    a, w = rnd((M, K), dtype, 6), rnd((N, K), dtype, 7)
    bias = rnd((N,), "float32", 8)
    out = torch.empty((M, N), dtype=DT[out_dtype], device=DEV)
    ops.gemm_plain(a, w, out, bias)
    ref = P.linear(a.cpu(), w.cpu(), bias.cpu())
    close(out, ref, out_dtype, scale=float(ref.abs().max()) + math.sqrt(K) * 1e-1)


def test_gemm_plain_rows_do_not_depend_on_the_batch():
    from libllm_b200.csrc import ops
    a, w = rnd((130, 300), "float32", 9), rnd((77, 300), "float32", 10)
    full = torch.empty((130, 77), device=DEV)
    one = torch.empty((1, 77), device=DEV)
    ops.gemm_plain(a, w, full)
    ops.gemm_plain(a[97:98], w, one)
    assert torch.equal(full[97:98], one)


def paged_cache(n_seqs, lens, n_kv, d, page, dtype, seed):
    """Random keys/values per sequence scattered over shuffled pages."""
    per = [(l + page - 1) // page for l in lens]
    n_pages = sum(per) + 3
    g = torch.Generator().manual_seed(seed)
    perm = torch.randperm(n_pages, generator=g).tolist()
    width = max(per) + 1
    table = torch.zeros((n_seqs, width), dtype=torch.int32)
    K = torch.full((n_pages, n_kv, page, d), 1e4).to(DT[dtype])     # unread places are poisoned
    V = torch.full((n_pages, n_kv, page, d), -1e4).to(DT[dtype])
    ks, vs = [], []
    o = 0
    for s, l in enumerate(lens):
        k = (torch.randn((l, n_kv, d), generator=g)).to(DT[dtype])
        v = (torch.randn((l, n_kv, d), generator=g)).to(DT[dtype])
        ks.append(k)
        vs.append(v)
        for lp in range(per[s]):
            pg = perm[o]
            o += 1
            table[s, lp] = pg
            n = min(page, l - lp * page)
            K[pg, :, :n] = k[lp * page:lp * page + n].transpose(0, 1)
            V[pg, :, :n] = v[lp * page:lp * page + n].transpose(0, 1)
    return K.to(DEV), V.to(DEV), table.to(DEV), ks, vs


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("n_heads,n_kv,d,window", [(4, 2, 16, None), (3, 1, 48, None), (8, 8, 128, None),
                                                     (6, 2, 256, None), (4, 1, 32, 37), (2, 2, 64, 64)])
def test_attention_generic(dtype, n_heads, n_kv, d, window):
    from libllm_b200.csrc import ops
    page = 16
    lens = [1, 70, 33, 130]
    q_lens = [1, 70, 5, 1]          # a whole prompt, the end of one, and single tokens
    K, V, table, ks, vs = paged_cache(4, lens, n_kv, d, page, dtype, 11)
    T = sum(q_lens)
    q = rnd((T, n_heads * d), dtype, 12)
    tok_seq = torch.tensor([s for s, n in enumerate(q_lens) for _ in range(n)], dtype=torch.int32, device=DEV)
    tok_pos = torch.tensor([lens[s] - n + i for s, n in enumerate(q_lens) for i in range(n)], dtype=torch.int32, device=DEV)
    out = torch.empty((T, n_heads * d), dtype=DT[dtype], device=DEV)
    scale = 1 / math.sqrt(d)
    ops.attention_generic(q, out, K, V, tok_seq, tok_pos, table, n_heads, n_kv, d, page, window, scale)
    o = 0
    for s, n in enumerate(q_lens):
        ref = P.attention_scores_softmax_values(q[o:o + n].cpu().view(n, n_heads, d), ks[s], vs[s], window)
        close(out[o:o + n].view(n, n_heads, d), ref, dtype, scale=1.0)
        o += n


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_attention_finds_one_far_key_among_hundreds(dtype):
    """Key 3 of 900 matches the query strongly; its value must dominate the output."""
    from libllm_b200.csrc import ops
    n_heads = n_kv = 1
    d, page, L = 64, 64, 900
    K, V, table, ks, vs = paged_cache(1, [L], n_kv, d, page, dtype, 13)
    q = rnd((1, d), dtype, 14)
    k3 = (q[0].float().cpu() * 3.0).to(DT[dtype])
    pg = int(table[0, 0])
    K[pg, 0, 3] = k3.to(DEV)
    ks[0][3, 0] = k3
    out = torch.empty((1, d), dtype=DT[dtype], device=DEV)
    pos = torch.tensor([L - 1], dtype=torch.int32, device=DEV)
    ops.attention_generic(q, out, K, V, torch.zeros(1, dtype=torch.int32, device=DEV), pos, table, 1, 1, d, page,
                          None, 1 / math.sqrt(d))
    ref = P.attention_scores_softmax_values(q.cpu().view(1, 1, d), ks[0], vs[0])
    close(out.view(1, 1, d), ref, dtype, scale=1.0)
    assert float((out.float().cpu()[0] - vs[0][3, 0].float()).abs().max()) < 0.2


@pytest.mark.parametrize("dtype,in_dtype", [("float32", "float32"), ("bfloat16", "bfloat16"), ("bfloat16", "float32")])
@pytest.mark.parametrize("n_heads,n_kv,d", [(4, 2, 16), (3, 1, 96)])
def test_rope_and_cache_write(dtype, in_dtype, n_heads, n_kv, d):
    from libllm_b200.csrc import ops
    from helpers import rotary_frequencies
    page, n_pages = 8, 12
    lens_past, q_lens = [0, 13, 40], [9, 1, 3]
    T = sum(q_lens)
    width = (n_heads + 2 * n_kv) * d
    qkv = rnd((T, width), in_dtype, 15)
    qkv0 = qkv.clone()
    q_out = torch.zeros((T, n_heads * d), dtype=DT[dtype], device=DEV)
    freqs = torch.tensor(rotary_frequencies(d, 10000.0, None), dtype=torch.float64)
    pos = torch.arange(64, dtype=torch.float64)
    ang = pos[:, None] * freqs[None]
    table = torch.cat([ang.cos(), ang.sin()], 1).float().to(DEV)
    tok_seq = torch.tensor([s for s, n in enumerate(q_lens) for _ in range(n)], dtype=torch.int32, device=DEV)
    tok_pos = torch.tensor([lens_past[s] + i for s, n in enumerate(q_lens) for i in range(n)], dtype=torch.int32, device=DEV)
    pt = torch.tensor([[3, 7, 0, 0, 0, 0], [1, 2, 0, 0, 0, 0], [4, 5, 6, 8, 9, 10]], dtype=torch.int32, device=DEV)
    K = torch.zeros((n_pages, n_kv, page, d), dtype=DT[dtype], device=DEV)
    V = torch.zeros_like(K)
    ops.rope_cache_write(qkv, q_out, n_heads, n_kv, d, table, tok_seq, tok_pos, pt, K, V, page)
    assert torch.equal(qkv, qkv0)
    x = qkv0.cpu().view(T, n_heads + 2 * n_kv, d)
    positions = tok_pos.cpu().to(torch.float64)
    qr = P.rope_rotate(x[:, :n_heads], positions, freqs)
    kr = P.rope_rotate(x[:, n_heads:n_heads + n_kv], positions, freqs)
    close(q_out.cpu().view(T, n_heads, d), qr, dtype)
    for t in range(T):
        s, p = int(tok_seq[t]), int(tok_pos[t])
        pg = int(pt[s, p // page])
        close(K[pg, :, p % page], kr[t], dtype)
        assert torch.equal(V[pg, :, p % page].cpu(), x[t, n_heads + n_kv:].to(DT[dtype]))
    # places no token was written to stay untouched
    written = {(int(pt[int(tok_seq[t]), int(tok_pos[t]) // page]), int(tok_pos[t]) % page) for t in range(T)}
    for pg in range(n_pages):
        for r in range(page):
            if (pg, r) not in written:
                assert float(K[pg, :, r].abs().max()) == 0.0


def test_argmax_and_ties():
    from libllm_b200.csrc import ops
    logits = rnd((5, 3001), "float32", 16)
    logits[1, 17] = logits[1, 2900] = 50.0          # tie: the lower index wins
    logits[2, 3000] = 60.0
    out = torch.empty(5, dtype=torch.int32, device=DEV)
    ops.argmax(logits, out)
    want = [P.sample_token(logits[i].cpu(), 0.0, 0, 1.0, 0.0) for i in range(5)]
    assert out.tolist() == want and want[1] == 17 and want[2] == 3000


def _interval_ok(logits_row, temperature, top_k, top_p, u, token):
    """``token`` is what the plain sampler returns for a number within 1e-5 of u."""
    return any(P.sample_token(logits_row, temperature, top_k, top_p, min(max(u + du, 0.0), 0.9999999)) == token
               for du in (0.0, -1e-5, 1e-5))


@pytest.mark.parametrize("vocab", [331, 128256])
@pytest.mark.parametrize("temperature,top_k,top_p", [(1.0, 50, 0.8), (0.7, 5, 1.0), (1.3, 1, 0.5), (0.8, 0, 1.0),
                                                      (1.0, 1024, 0.95)])
def test_sampling_matches_plain_sampler(vocab, temperature, top_k, top_p):
    from libllm_b200.csrc import ops
    B = 6
    logits = rnd((B, vocab), "float32", 17, 3.0)
    logits[0, 5] = logits[0, 9] = logits[0].max() + 1.0        # tied leaders
    us = [0.0, 0.1234, 0.5, 0.77, 0.999, 0.31]
    uni = torch.tensor(us, dtype=torch.float32, device=DEV)
    out = torch.empty(B, dtype=torch.int32, device=DEV)
    ops.sample(logits, temperature, top_k, top_p, uni, out)
    for i in range(B):
        assert _interval_ok(logits[i].cpu(), temperature, min(top_k, vocab), top_p, us[i], int(out[i])), (i, int(out[i]))
    # a row's draw does not depend on its neighbours
    out1 = torch.empty(1, dtype=torch.int32, device=DEV)
    ops.sample(logits[3:4], temperature, top_k, top_p, uni[3:4], out1)
    assert int(out1[0]) == int(out[3])
    # temperature 0 is argmax
    ops.sample(logits, 0.0, top_k, top_p, uni, out)
    want = logits.argmax(-1).tolist()
    want[0] = 5                                  # tied leaders: the lower index wins
    assert out.tolist() == want


@pytest.mark.parametrize("case", ["flat", "many_tied_leaders", "ties_at_the_kth", "none_near_the_maximum"])
def test_sampling_rows_that_the_quick_selection_must_get_right_or_hand_on(case):
    """Rows at the edges of the two ways the kernel finds the top_k: all logits equal and thousands
    of tied leaders (more candidates than the quick selection sorts), ties exactly at the k-th place
    inside it (the lower indices are taken), and fewer than top_k logits near the maximum."""
    from libllm_b200.csrc import ops
    V, top_k = 20000, 50
    g = torch.Generator().manual_seed(23)
    if case == "flat":
        row = torch.full((V,), 1.5)
    elif case == "many_tied_leaders":
        row = torch.randn(V, generator=g) - 30.0
        row[torch.randperm(V, generator=g)[:3000]] = 4.0
    elif case == "ties_at_the_kth":
        row = torch.randn(V, generator=g) - 40.0
        idx = torch.randperm(V, generator=g)
        row[idx[:10]] = torch.linspace(5.0, 6.0, 10)
        row[idx[10:1510]] = 4.0
    else:
        row = torch.randn(V, generator=g) * 0.1 - 50.0
        row[torch.randperm(V, generator=g)[:7]] = torch.linspace(1.0, 3.0, 7)
    us = [0.0, 0.21, 0.5, 0.83, 0.97, 0.9999]
    logits = row.to(DEV).repeat(len(us), 1).contiguous()
    uni = torch.tensor(us, dtype=torch.float32, device=DEV)
    out = torch.empty(len(us), dtype=torch.int32, device=DEV)
    for temperature, top_p in ((1.0, 1.0), (0.7, 0.9)):
        ops.sample(logits, temperature, top_k, top_p, uni, out)
        for i, u in enumerate(us):
            assert _interval_ok(row, temperature, top_k, top_p, u, int(out[i])), (case, temperature, top_p, u, int(out[i]))


def test_kernels_refuse_what_they_cannot_do():
    from libllm_b200.csrc import ops
    from libllm_b200.errors import ExtensionError, UnsupportedError
    with pytest.raises(ExtensionError):
        ops.swiglu(torch.zeros(2, 4), torch.zeros(2, 2))          # host tensors: no CPU fallback
    logits = rnd((1, 100), "float32", 18)
    with pytest.raises(UnsupportedError):
        ops.sample(logits, 1.0, 5000, 1.0, torch.zeros(1, device=DEV), torch.zeros(1, dtype=torch.int32, device=DEV))


@pytest.mark.parametrize("out_dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("M,N,K", [(1, 96, 64), (8, 200, 80), (3, 331, 176), (16, 2048, 2048), (33, 130, 520),
                                   (64, 1000, 4096), (7, 17, 8)])
def test_small_batch_product(out_dtype, M, N, K):
    from libllm_b200.csrc import ops
    x, w = rnd((M, K), "bfloat16", 20), rnd((N, K), "bfloat16", 21, 0.05)
    out = torch.empty((M, N), dtype=DT[out_dtype], device=DEV)
    ops.gemv_bf16(x, w, out)
    ref = P.linear(x.cpu(), w.cpu())
    close(out, ref, out_dtype, scale=float(ref.abs().max()))
    # one token's result does not depend on the others in the batch: bit for bit when the
    # batch has the same size, to rounding when the size (and with it the K split) differs
    x2 = rnd((M, K), "bfloat16", 99)
    x2[M - 1] = x[M - 1]
    out2 = torch.empty((M, N), dtype=DT[out_dtype], device=DEV)
    ops.gemv_bf16(x2, w, out2)
    assert torch.equal(out2[M - 1], out[M - 1])
    one = torch.empty((1, N), dtype=DT[out_dtype], device=DEV)
    ops.gemv_bf16(x[M - 1:M], w, one)
    close(one, ref[M - 1:M], out_dtype, scale=float(ref.abs().max()))


@pytest.mark.parametrize("M,I,K", [(1, 96, 64), (5, 173, 80), (8, 8192, 2048), (40, 300, 256)])
def test_small_batch_product_with_swiglu(M, I, K):
    from libllm_b200.csrc import ops
    x, w = rnd((M, K), "bfloat16", 22), rnd((2 * I, K), "bfloat16", 23, 0.2)
    out = torch.empty((M, I), dtype=torch.bfloat16, device=DEV)
    ops.gemv_bf16(x, w, out, swiglu=True)
    gu = P.linear(x.cpu(), w.cpu())
    close(out, P.swiglu(gu[:, :I], gu[:, I:]), "bfloat16")


@pytest.mark.parametrize("n_heads,n_kv,d,window", [(4, 2, 16, None), (3, 1, 32, None), (32, 8, 64, None),
                                                     (8, 1, 128, None), (8, 8, 64, None), (6, 2, 128, 100)])
@pytest.mark.parametrize("chunk,n_splits", [(64, 16), (192, 6), (1024, 1)])
def test_attention_decode(n_heads, n_kv, d, window, chunk, n_splits):
    from libllm_b200.csrc import ops
    page = 64
    lens = [1, 70, 333, 1000, 64]
    B = len(lens)
    K, V, table, ks, vs = paged_cache(B, lens, n_kv, d, page, "bfloat16", 24)
    q = rnd((B, n_heads * d), "bfloat16", 25)
    pos = torch.tensor([l - 1 for l in lens], dtype=torch.int32, device=DEV)
    out = torch.empty((B, n_heads * d), dtype=torch.bfloat16, device=DEV)
    ws_o = torch.full((B * n_heads * n_splits * d,), float("nan"), device=DEV)
    ws_ml = torch.full((B * n_heads * n_splits * 2,), float("nan"), device=DEV)
    assert ops.attention_decode_supported(d, n_heads // n_kv)
    ops.attention_decode(q, out, K, V, pos, table, n_heads, n_kv, d, page, chunk, n_splits, window, 1 / math.sqrt(d),
                         ws_o, ws_ml)
    for b in range(B):
        ref = P.attention_scores_softmax_values(q[b:b + 1].cpu().view(1, n_heads, d), ks[b], vs[b], window)
        close(out[b].view(1, n_heads, d), ref, "bfloat16", scale=1.0)


def prefill_inputs(lens, q_lens):
    start = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32, device=DEV)
    past = torch.tensor([l - n for l, n in zip(lens, q_lens)], dtype=torch.int32, device=DEV)
    return start, past


@pytest.mark.parametrize("n_heads,n_kv,d,window", [(4, 2, 16, None), (3, 1, 48, None), (32, 8, 64, None),
                                                     (5, 5, 80, None), (8, 2, 128, None), (4, 1, 32, 37),
                                                     (2, 2, 64, 64), (6, 3, 112, 130)])
def test_attention_prefill(n_heads, n_kv, d, window):
    """Whole prompts, the end of a prompt behind cached tokens, tile edges (63, 64, 65 rows) and
    single tokens in one launch, against the plain attention of each sequence."""
    from libllm_b200.csrc import ops
    page = 64
    lens = [1, 70, 333, 200, 64, 65, 63]
    q_lens = [1, 70, 5, 150, 64, 65, 1]
    B = len(lens)
    K, V, table, ks, vs = paged_cache(B, lens, n_kv, d, page, "bfloat16", 31)
    T = sum(q_lens)
    q = rnd((T, n_heads * d), "bfloat16", 32)
    out = torch.full((T, n_heads * d), float("nan"), dtype=torch.bfloat16, device=DEV)
    start, past = prefill_inputs(lens, q_lens)
    assert ops.attention_prefill_supported(d, page)
    ops.attention_prefill(q, out, K, V, start, past, table, B, max(q_lens), n_heads, n_kv, d, page, window,
                          1 / math.sqrt(d))
    o = 0
    for s, n in enumerate(q_lens):
        ref = P.attention_scores_softmax_values(q[o:o + n].cpu().view(n, n_heads, d), ks[s], vs[s], window)
        close(out[o:o + n].view(n, n_heads, d), ref, "bfloat16", scale=1.0)
        o += n


def test_attention_prefill_finds_a_far_key_and_respects_the_window_edge():
    """Row 700 of a 900-token prompt matches key 3 strongly: without a window key 3's value
    dominates that row; with a window of 697 key 3 is the last one outside (700 - 697 = 3) and
    must not be seen, with 698 it is the first one inside."""
    from libllm_b200.csrc import ops
    d, page, L = 64, 64, 900
    K, V, table, ks, vs = paged_cache(1, [L], 1, d, page, "bfloat16", 33)
    q = rnd((L, d), "bfloat16", 34)
    k3 = (q[700].float().cpu() * 3.0).to(torch.bfloat16)
    K[int(table[0, 0]), 0, 3] = k3.to(DEV)
    ks[0][3, 0] = k3
    start, past = prefill_inputs([L], [L])
    for window, sees in ((None, True), (697, False), (698, True)):
        out = torch.empty((L, d), dtype=torch.bfloat16, device=DEV)
        ops.attention_prefill(q, out, K, V, start, past, table, 1, L, 1, 1, d, page, window, 1 / math.sqrt(d))
        ref = P.attention_scores_softmax_values(q.cpu().view(L, 1, d), ks[0], vs[0], window)
        close(out.view(L, 1, d), ref, "bfloat16", scale=1.0)
        near = float((out[700].float().cpu() - vs[0][3, 0].float()).abs().max()) < 0.2
        assert near == sees, (window, near)


def test_attention_prefill_refuses_what_it_cannot_do():
    from libllm_b200.csrc import ops
    from libllm_b200.errors import UnsupportedError
    assert not ops.attention_prefill_supported(256, 64) and not ops.attention_prefill_supported(64, 16)
    assert not ops.attention_prefill_supported(40, 64)
    K, V, table, _, _ = paged_cache(1, [10], 1, 144, 64, "bfloat16", 35)
    q = rnd((10, 144), "bfloat16", 36)
    start, past = prefill_inputs([10], [10])
    with pytest.raises(UnsupportedError):
        ops.attention_prefill(q, torch.empty_like(q), K, V, start, past, table, 1, 10, 1, 1, 144, 64, None, 0.1)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_rope_on_a_part_of_the_channels(dtype):
    """Only the first 16 of 32 channels rotate (pairs (i, i + 8)); the rest pass through.  This is
    the general kernel; heads that rotate whole take the vectorised one."""
    from libllm_b200.csrc import ops
    n_heads, n_kv, d, rot, page = 2, 1, 32, 16, 8
    T = 5
    qkv = rnd((T, (n_heads + 2 * n_kv) * d), dtype, 40)
    q_out = torch.zeros((T, n_heads * d), dtype=DT[dtype], device=DEV)
    freqs = torch.tensor([0.5 ** i for i in range(rot // 2)], dtype=torch.float64)
    ang = torch.arange(16, dtype=torch.float64)[:, None] * freqs[None]
    table = torch.cat([ang.cos(), ang.sin()], 1).float().to(DEV)
    tok_seq = torch.zeros(T, dtype=torch.int32, device=DEV)
    tok_pos = torch.arange(3, 3 + T, dtype=torch.int32, device=DEV)
    pt = torch.tensor([[2, 0, 1, 3]], dtype=torch.int32, device=DEV)
    K = torch.zeros((4, n_kv, page, d), dtype=DT[dtype], device=DEV)
    V = torch.zeros_like(K)
    ops.rope_cache_write(qkv, q_out, n_heads, n_kv, d, table, tok_seq, tok_pos, pt, K, V, page)
    x = qkv.cpu().view(T, n_heads + 2 * n_kv, d)
    want = x[:, :n_heads].clone().double()
    want[..., :rot] = P.rope_rotate(x[:, :n_heads, :rot], tok_pos.cpu().double(), freqs)
    close(q_out.cpu().view(T, n_heads, d), want, dtype)
    kwant = x[:, n_heads:n_heads + n_kv].clone().double()
    kwant[..., :rot] = P.rope_rotate(x[:, n_heads:n_heads + n_kv, :rot], tok_pos.cpu().double(), freqs)
    for t in range(T):
        p = 3 + t
        close(K[int(pt[0, p // page]), :, p % page], kwant[t], dtype)


TC_SHAPES = [(1, 128, 64), (8, 200, 80), (3, 331, 176), (16, 2048, 2048), (17, 130, 520), (64, 300, 128),
             (100, 256, 192), (300, 500, 72), (8, 3072, 2048), (2, 64, 8)]


@pytest.mark.parametrize("out_dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("M,N,K", TC_SHAPES)
def test_tensor_core_product(out_dtype, M, N, K):
    """Sizes that are no multiple of any tile (rows of W, tokens, K), one token, many tokens."""
    from libllm_b200.csrc import ops
    x = rnd((M, K), "bfloat16", 50)
    w = rnd((N, K), "bfloat16", 51, std=0.1)
    out = torch.full((M, N), float("nan"), dtype=DT[out_dtype], device=DEV)
    assert ops.gemm_tc_supported(x, w)
    ops.gemm_tc(x, w, out)
    ops.check_tc_status()
    close(out, P.linear(x.cpu(), w.cpu()), "bfloat16" if out_dtype == "bfloat16" else "float32",
          scale=None if out_dtype == "bfloat16" else 50 * float(P.linear(x.cpu(), w.cpu()).abs().max()))


@pytest.mark.parametrize("M,N,K,parts", [(8, 2048, 2048, 4), (5, 200, 8192, 8), (40, 130, 520, 2), (16, 2048, 8192, 8)])
def test_tensor_core_product_in_parts_of_k(M, N, K, parts):
    from libllm_b200.csrc import ops
    x = rnd((M, K), "bfloat16", 52)
    w = rnd((N, K), "bfloat16", 53, std=0.1)
    out = torch.full((parts, M, N), float("nan"), dtype=torch.float32, device=DEV)
    ops.gemm_tc(x, w, out)
    ops.check_tc_status()
    ref = P.linear(x.cpu(), w.cpu())
    close(out.sum(0), ref, "float32", scale=50 * float(ref.abs().max()))
    assert 1 <= ops.gemm_tc_suggest_parts(M, N, K) <= 8


@pytest.mark.parametrize("M,I,K", [(1, 64, 64), (5, 173, 80), (8, 8192, 2048), (40, 300, 256), (200, 128, 136), (257, 391, 200),
                                   (1000, 1024, 512)])
def test_tensor_core_product_with_swiglu(M, I, K):
    from libllm_b200.csrc import ops
    x = rnd((M, K), "bfloat16", 54)
    w = rnd((2 * I, K), "bfloat16", 55, std=0.1)
    out = torch.full((M, I), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.gemm_tc(x, w, out, swiglu=True)
    ops.check_tc_status()
    gu = P.linear(x.cpu(), w.cpu())
    close(out, P.swiglu(gu[:, :I], gu[:, I:]), "bfloat16")


def test_tensor_core_product_rows_do_not_depend_on_the_batch():
    """A token's row is the same alone and among 200 others: each token is its own column of the tile."""
    from libllm_b200.csrc import ops
    x = rnd((200, 256), "bfloat16", 56)
    w = rnd((384, 256), "bfloat16", 57, std=0.1)
    full = torch.empty((200, 384), dtype=torch.float32, device=DEV)
    ops.gemm_tc(x, w, full)
    for r in (0, 17, 199):
        one = torch.empty((1, 384), dtype=torch.float32, device=DEV)
        ops.gemm_tc(x[r:r + 1].contiguous(), w, one)
        assert torch.equal(one[0], full[r])
    ops.check_tc_status()


@pytest.mark.parametrize("n_heads,n_kv,d,window", [(4, 2, 16, None), (3, 1, 32, None), (32, 8, 64, None), (8, 1, 128, None),
                                                     (8, 8, 64, None), (6, 2, 128, 100), (10, 2, 48, None)])
# up to 16 splits are joined through a cluster's shared memory, more through scratch in global memory;
# chunk 0: each length cut into 5 runs
@pytest.mark.parametrize("chunk,n_splits", [(64, 16), (64, 18), (192, 6), (1024, 1), (0, 5)])
def test_attention_decode_fused(n_heads, n_kv, d, window, chunk, n_splits):
    """Rotation, cache append, attention and the joining of splits in one launch: the outputs
    against the plain rotation + attention, the cache rows it must have written, and a second
    launch one position later (the counters must have come back to zero)."""
    from libllm_b200.csrc import ops
    from helpers import rotary_frequencies
    page = 64
    lens = [1, 70, 333, 1000, 64, 65]        # cached tokens, the new one included
    B = len(lens)
    K, V, table_pt, ks, vs = paged_cache(B, [l + 1 for l in lens], n_kv, d, page, "bfloat16", 60)
    freqs = torch.tensor(rotary_frequencies(d, 10000.0, None), dtype=torch.float64)
    ang = torch.arange(1100, dtype=torch.float64)[:, None] * freqs[None]
    table = torch.cat([ang.cos(), ang.sin()], 1).float().to(DEV)
    counters = torch.zeros(B * n_kv, dtype=torch.int32, device=DEV)
    for step in range(2):
        pos = [l - 1 + step for l in lens]
        gen = torch.Generator().manual_seed(61 + step)
        if step == 0:
            qkv = torch.randn((B, (n_heads + 2 * n_kv) * d), generator=gen).to(DEV)
            qkv_in = qkv
        else:       # the stacked product in three parts over K, which the kernel adds in order
            qkv_in = torch.randn((3, B, (n_heads + 2 * n_kv) * d), generator=gen).to(DEV)
            qkv = (qkv_in[0] + qkv_in[1]) + qkv_in[2]
        out = torch.full((B, n_heads * d), float("nan"), dtype=torch.bfloat16, device=DEV)
        ws_o = torch.full((B * n_heads * n_splits * d,), float("nan"), device=DEV)
        ws_ml = torch.full((B * n_heads * n_splits * 2,), float("nan"), device=DEV)
        tok_pos = torch.tensor(pos, dtype=torch.int32, device=DEV)
        assert ops.attention_decode_tc_supported(d, page, n_heads // n_kv)
        ops.attention_decode_tc(qkv_in, out, table, K, V, tok_pos, table_pt, n_heads, n_kv, d, page, chunk, n_splits, window,
                                1 / math.sqrt(d), True, ws_o, ws_ml, counters, max_len=1100)
        assert int(counters.abs().sum()) == 0
        x = qkv.cpu().view(B, n_heads + 2 * n_kv, d)
        for b in range(B):
            p = torch.tensor([pos[b]], dtype=torch.float64)
            q = P.rope_rotate(x[b:b + 1, :n_heads], p, freqs).to(torch.bfloat16)
            k_new = P.rope_rotate(x[b:b + 1, n_heads:n_heads + n_kv], p, freqs).to(torch.bfloat16)
            v_new = x[b:b + 1, n_heads + n_kv:].to(torch.bfloat16)
            # the plain side's cache: the rows before the new token as they were, then the new one
            ks[b][pos[b]] = k_new[0]
            vs[b][pos[b]] = v_new[0]
            pg = int(table_pt[b, pos[b] // page])
            assert torch.equal(K[pg, :, pos[b] % page].cpu(), k_new[0]) or \
                float((K[pg, :, pos[b] % page].cpu().float() - k_new[0].float()).abs().max()) <= 2 ** -7 * float(k_new.abs().max())
            assert torch.equal(V[pg, :, pos[b] % page].cpu(), v_new[0])
            ref = P.attention_scores_softmax_values(q, ks[b][:pos[b] + 1], vs[b][:pos[b] + 1], window)
            # bfloat16 rounds relative to the value: a sequence of one or two keys returns values of up to 4
            close(out[b].view(1, n_heads, d), ref, "bfloat16", scale=max(1.0, float(ref.abs().max())))


@pytest.mark.parametrize("n_heads,n_kv,d,window", [(32, 8, 64, None), (3, 1, 64, None), (8, 2, 128, None), (2, 2, 64, 64),
                                                     (6, 3, 128, 130), (4, 1, 64, 37)])
@pytest.mark.parametrize("form", [1, 2])
def test_attention_prefill_on_tcgen05(n_heads, n_kv, d, window, form):
    """The tcgen05 kernel on the cases of the mma.sync one: whole prompts, the end of a prompt behind
    cached tokens, tile edges (127, 128, 129 rows), single tokens, windows."""
    from libllm_b200.csrc import ops
    page = 64
    lens = [1, 70, 333, 200, 128, 129, 127, 300]
    q_lens = [1, 70, 5, 150, 128, 129, 1, 300]
    B = len(lens)
    K, V, table, ks, vs = paged_cache(B, lens, n_kv, d, page, "bfloat16", 71)
    T = sum(q_lens)
    q = rnd((T, n_heads * d), "bfloat16", 72)
    out = torch.full((T, n_heads * d), float("nan"), dtype=torch.bfloat16, device=DEV)
    start, past = prefill_inputs(lens, q_lens)
    assert ops.attention_prefill_tc_supported(d, page)
    ops.attention_prefill_tc(q, out, K, V, start, past, table, B, max(q_lens), n_heads, n_kv, d, page, window,
                             1 / math.sqrt(d), form)
    ops.check_tc_status()
    o = 0
    for s, n in enumerate(q_lens):
        ref = P.attention_scores_softmax_values(q[o:o + n].cpu().view(n, n_heads, d), ks[s], vs[s], window)
        close(out[o:o + n].view(n, n_heads, d), ref, "bfloat16", scale=max(1.0, float(ref.abs().max())))
        o += n


@pytest.mark.parametrize("form", [1, 2])
def test_attention_prefill_on_tcgen05_finds_a_far_key_and_respects_the_window_edge(form):
    from libllm_b200.csrc import ops
    d, page, L = 64, 64, 900
    K, V, table, ks, vs = paged_cache(1, [L], 1, d, page, "bfloat16", 73)
    q = rnd((L, d), "bfloat16", 74)
    k3 = (q[700].float().cpu() * 3.0).to(torch.bfloat16)
    K[int(table[0, 0]), 0, 3] = k3.to(DEV)
    ks[0][3, 0] = k3
    start, past = prefill_inputs([L], [L])
    for window, sees in ((None, True), (697, False), (698, True)):
        out = torch.empty((L, d), dtype=torch.bfloat16, device=DEV)
        ops.attention_prefill_tc(q, out, K, V, start, past, table, 1, L, 1, 1, d, page, window, 1 / math.sqrt(d), form)
        ops.check_tc_status()
        ref = P.attention_scores_softmax_values(q.cpu().view(L, 1, d), ks[0], vs[0], window)
        close(out.view(L, 1, d), ref, "bfloat16", scale=max(1.0, float(ref.abs().max())))
        near = float((out[700].float().cpu() - vs[0][3, 0].float()).abs().max()) < 0.2
        assert near == sees, (window, near)


@pytest.mark.parametrize("d", [64, 128])
@pytest.mark.parametrize("step_nats", [6.5, 2.0, -6.5])
@pytest.mark.parametrize("form", [1, 2])
def test_attention_prefill_on_tcgen05_when_the_maximum_moves_from_tile_to_tile(d, step_nats, form):
    """The kernel moves a row's exponent reference only when a tile's maximum exceeds it by 2^8, and
    then rescales the output row in tensor memory.  Random scores settle the reference in the first
    tile; here every 64 keys the scores step up by 6.5 nats (the reference moves in every tile and
    earlier tiles all but vanish), by 2 nats (it lags behind the maximum, moving every third tile or
    so, and the probabilities in between exceed 1), or down (it never moves after the first tile)."""
    from libllm_b200.csrc import ops
    page, L, n_heads, n_kv = 64, 700, 2, 1
    K, V, table, ks, vs = paged_cache(1, [L], n_kv, d, page, "bfloat16", 75)
    q = rnd((L, n_heads * d), "bfloat16", 76, 0.3)
    q.view(L, n_heads, d)[:, :, 0] = math.sqrt(d)              # channel 0 alone gives key j's score k[j, 0]
    k = ks[0][:, 0].float() * 0.3
    k[:, 0] = step_nats * (torch.arange(L) // 64).float()
    ks[0][:, 0] = k.to(torch.bfloat16)
    for lp in range((L + page - 1) // page):
        n = min(page, L - lp * page)
        K[int(table[0, lp]), 0, :n] = ks[0][lp * page:lp * page + n, 0].to(DEV)
    start, past = prefill_inputs([L], [L])
    out = torch.full((L, n_heads * d), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.attention_prefill_tc(q, out, K, V, start, past, table, 1, L, n_heads, n_kv, d, page, None, 1 / math.sqrt(d), form)
    ops.check_tc_status()
    ref = P.attention_scores_softmax_values(q.cpu().view(L, n_heads, d), ks[0], vs[0], None)
    close(out.view(L, n_heads, d), ref, "bfloat16", scale=max(1.0, float(ref.abs().max())))


@pytest.mark.parametrize("d,n_heads,n_kv", [(64, 32, 8), (128, 8, 2)])
@pytest.mark.parametrize("form", [1, 2])
def test_attention_prefill_on_tcgen05_with_a_prompt_of_2048_tokens(d, n_heads, n_kv, form):
    """A prompt as long as the benchmark's: 16 query tiles a head and up to 32 key tiles a CTA, so the
    rings of key/value stages and the two score buffers go round many times, with queries that lie
    strided in the stacked q|k|v rows as the engine has them.  Every 97th row is checked against
    the plain attention."""
    from libllm_b200.csrc import ops
    page, L = 64, 2048
    K, V, table, ks, vs = paged_cache(1, [L], n_kv, d, page, "bfloat16", 81)
    qkv = rnd((L, (n_heads + 2 * n_kv) * d), "bfloat16", 82)
    q = qkv[:, :n_heads * d]
    start, past = prefill_inputs([L], [L])
    out = torch.full((L, n_heads * d), float("nan"), dtype=torch.bfloat16, device=DEV)
    for _ in range(3):          # the same launch again: a race shows in some runs only
        ops.attention_prefill_tc(q, out, K, V, start, past, table, 1, L, n_heads, n_kv, d, page, None, 1 / math.sqrt(d), form)
        ops.check_tc_status()
        assert bool(torch.isfinite(out.float()).all())
        rows = list(range(0, L, 97)) + [L - 1]
        qs = q[rows].cpu().view(len(rows), n_heads, d)
        for i, r in enumerate(rows):
            ref = P.attention_scores_softmax_values(qs[i:i + 1], ks[0][:r + 1], vs[0][:r + 1], None)
            close(out[r].view(1, n_heads, d), ref, "bfloat16", scale=max(1.0, float(ref.abs().max())))


def test_copy_words_between_pinned_host_memory_and_the_device():
    """The small copies inside a single-token step's graph are kernels that read and write pinned
    host memory directly: both directions, an odd count, and a refusal of pageable memory."""
    from libllm_b200.csrc import ops
    from libllm_b200.errors import ExtensionError
    n = 2353
    host = torch.arange(n, dtype=torch.int32).pin_memory()
    dev = torch.full((n + 7,), -1, dtype=torch.int32, device=DEV)
    ops.copy_words(host, dev, n)
    torch.cuda.synchronize()
    assert torch.equal(dev[:n].cpu(), host) and bool((dev[n:] == -1).all())
    back = torch.zeros(n, dtype=torch.int32).pin_memory()
    ops.copy_words(dev * 3, back, n)
    torch.cuda.synchronize()
    assert torch.equal(back, host * 3)
    with pytest.raises(ExtensionError):
        ops.copy_words(torch.zeros(4, dtype=torch.int32), dev, 4)


# ---------------------------------------------------------------- a chain of products and norms in one launch
def _chain_case(T, Kq, H, inter, V, parts_o, parts_d, seed, repeats=3):
    from libllm_b200.csrc import ops
    eps = 3e-5
    x0 = rnd((T, Kq), "bfloat16", seed)
    wo = rnd((H, Kq), "bfloat16", seed + 1, Kq ** -0.5)
    wgu = rnd((2 * inter, H), "bfloat16", seed + 2, H ** -0.5)
    wd = rnd((H, inter), "bfloat16", seed + 3, inter ** -0.5)
    wh = rnd((V, H), "bfloat16", seed + 4, H ** -0.5)
    n1 = (1 + 0.1 * rnd((H,), "float32", seed + 5))
    n2 = (1 + 0.1 * rnd((H,), "float32", seed + 6))
    resid0 = rnd((T, H), "float32", seed + 7)
    rows = torch.tensor([T - 1, 0, T // 2][:min(3, T)], dtype=torch.int32, device=DEV)
    W = rows.numel()

    # the plain computation, rounding to bfloat16 where the chain does
    def norm(v, w):
        return (v * w * torch.rsqrt((v * v).mean(-1, keepdim=True) + eps)).to(torch.bfloat16)
    o = x0.float() @ wo.float().T
    v1 = resid0 + o
    h1 = norm(v1, n1)
    gu = h1.float() @ wgu.float().T
    m = (torch.nn.functional.silu(gu[:, :inter]) * gu[:, inter:]).to(torch.bfloat16)
    d = m.float() @ wd.float().T
    v2 = v1 + d
    h2 = norm(v2[rows.long()], n2)
    logits_ref = h2.float() @ wh.float().T

    counters = torch.zeros(16, dtype=torch.int32, device=DEV)
    for _ in range(repeats):
        resid = resid0.clone()
        o_parts = torch.full((parts_o, T, H), float("nan"), dtype=torch.float32, device=DEV)
        h1_out = torch.empty((T, H), dtype=torch.bfloat16, device=DEV)
        m_out = torch.empty((T, inter), dtype=torch.bfloat16, device=DEV)
        d_parts = torch.full((parts_d, T, H), float("nan"), dtype=torch.float32, device=DEV)
        h2_out = torch.empty((W, H), dtype=torch.bfloat16, device=DEV)
        logits = torch.full((W, V), float("nan"), dtype=torch.float32, device=DEV)
        jobs = [
            ops.chain_product(x0, wo, o_parts),
            ops.chain_norm(resid, o_parts, n1, eps, h1_out, deps=(0, -1)),
            ops.chain_product(h1_out, wgu, m_out, swiglu=True, deps=(1, -1)),
            ops.chain_product(m_out, wd, d_parts, deps=(2, -1)),
            ops.chain_norm(resid, d_parts, n2, eps, h2_out, rows=rows, deps=(3, 1)),
            ops.chain_product(h2_out, wh, logits, deps=(4, -1)),
        ]
        ops.gemm_chain(jobs, counters)
        torch.cuda.synchronize()
        ops.check_tc_status()
        assert int(counters.abs().sum()) == 0, "the chain left its counters non-zero"
        close(resid, v1, "bfloat16")
        close(h1_out.float(), h1.float(), "bfloat16")
        close(m_out.float(), m.float(), "bfloat16")
        close(h2_out.float(), h2.float(), "bfloat16")
        close(logits, logits_ref, "bfloat16")


@pytest.mark.parametrize("T,Kq,H,inter,V,parts_o,parts_d", [
    (5, 136, 200, 328, 1000, 2, 3),          # sizes that are no power of two, few tiles
    (16, 512, 1024, 2816, 20000, 4, 8),      # several tiles per CTA and job
    (23, 264, 520, 1096, 3001, 1, 2),        # 32-token shape, one part
    (40, 512, 1024, 1536, 9000, 2, 4),       # 64-token shape
    (1, 2048, 2048, 8192, 32000, 8, 8),      # the engine's widths at batch 1
])
def test_gemm_chain_layer(T, Kq, H, inter, V, parts_o, parts_d):
    _chain_case(T, Kq, H, inter, V, parts_o, parts_d, seed=11)


def test_gemm_chain_refuses():
    from libllm_b200.csrc import ops
    from libllm_b200.errors import UnsupportedError
    counters = torch.zeros(16, dtype=torch.int32, device=DEV)
    x = rnd((65, 64), "bfloat16", 1)
    w = rnd((128, 64), "bfloat16", 2)
    out = torch.empty((65, 128), dtype=torch.float32, device=DEV)
    with pytest.raises(UnsupportedError):
        ops.gemm_chain([ops.chain_product(x, w, out)], counters)          # more tokens than a chain takes
    x = rnd((4, 64), "bfloat16", 1)
    out = torch.empty((4, 128), dtype=torch.float32, device=DEV)
    with pytest.raises(UnsupportedError):
        ops.gemm_chain([ops.chain_product(x, w, out, deps=(0, -1))], counters)   # depends on itself
    with pytest.raises(UnsupportedError):
        ops.gemm_chain([ops.chain_product(x, w, out)] * 9, counters)      # more jobs than one launch holds
