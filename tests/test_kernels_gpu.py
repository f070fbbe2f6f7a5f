"""Each kernel alone against a plain PyTorch reference of the same operation,
at sizes other than the engine's test models: widths and vocabularies that are
no power of two, head sizes in steps of 16, odd numbers of heads and groups."""
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def _ops():
    from sglang_c_b200.csrc import ops
    return ops


def _rand(*shape, dtype=torch.float32, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype).to(DEV)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,E,V,P", [(1, 48, 11, 5), (37, 1600, 1000, 300), (5, 100, 50257, 64)])
def test_embed(T, E, V, P, dtype):
    ops = _ops()
    wte, wpe = _rand(V, E, dtype=dtype, seed=1), _rand(P, E, dtype=dtype, seed=2)
    g = torch.Generator().manual_seed(3)
    tok = torch.randint(0, V, (T,), generator=g, dtype=torch.int32).to(DEV)
    pos = torch.randint(0, P, (T,), generator=g, dtype=torch.int32).to(DEV)
    out = torch.empty(T, E, device=DEV)
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    ops.embed(tok, wte, out, positions=pos, pos_table=wpe, err_flag=err)
    ref = wte.float()[tok.long()] + wpe.float()[pos.long()]
    assert torch.equal(out, ref) and int(err.item()) == 0
    out2 = torch.empty(T, E, device=DEV)
    ops.embed(tok, wte, out2)
    ops.add_rows(out2, pos, wpe)
    assert torch.equal(out2, ref)
    # an id outside the table is flagged, not read
    tok[0] = V
    ops.embed(tok, wte, out, positions=pos, pos_table=wpe, err_flag=err)
    assert int(err.item()) == 1 and float(out[0].abs().max()) == 0.0


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n,E,eps", [(1, 16, 1e-5), (33, 96, 1e-6), (7, 1600, 1e-5), (3, 50, 1e-3), (2, 4099, 1e-5),
                                     (1300, 768, 1e-5), (1025, 1600, 1e-5), (1100, 96, 1e-6), (1024, 2048, 1e-5), (2000, 24, 1e-5)])
def test_layernorm(n, E, eps, out_dtype):
    ops = _ops()
    x = _rand(n, E, seed=4, scale=3.0) + 1.5
    gamma, beta = _rand(E, seed=5) + 1.0, _rand(E, seed=6)
    out = torch.empty(n, E, dtype=out_dtype, device=DEV)
    ops.layernorm(x, gamma, beta, eps, out)
    xd = x.double()
    ref = (xd - xd.mean(-1, keepdim=True)) / torch.sqrt(xd.var(-1, unbiased=False, keepdim=True) + eps)
    ref = ref * gamma.double() + beta.double()
    tol = 2e-5 if out_dtype == torch.float32 else 4e-2
    assert float((out.double() - ref).abs().max()) < tol
    # gathered rows
    rows = torch.tensor(list(range(n - 1, -1, -1)), dtype=torch.int32, device=DEV)
    out2 = torch.empty(n, E, dtype=out_dtype, device=DEV)
    ops.layernorm(x, gamma, beta, eps, out2, rows=rows)
    assert torch.equal(out2, out.flip(0))


@pytest.mark.parametrize("in_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("M,N,K", [(1, 1, 1), (5, 70, 33), (65, 129, 100), (130, 50257 // 16, 96), (3, 320, 1600),
                                   (16, 1571, 772), (9, 40, 4), (1500, 1200, 200), (1155, 2304, 100)])
def test_gemm_simt(M, N, K, in_dtype):
    ops = _ops()
    a, w, bias = _rand(M, K, dtype=in_dtype, seed=7), _rand(N, K, dtype=in_dtype, seed=8, scale=0.1), _rand(N, seed=9)
    ref = a.double() @ w.double().t() + bias.double()
    tol = 1e-5 * math.sqrt(K) if in_dtype == torch.float32 else 1e-4 * math.sqrt(K)
    out = torch.empty(M, N, device=DEV)
    ops.gemm_simt(a, w, bias, out=out)
    assert float((out.double() - ref).abs().max()) < tol
    for act, fn in (("gelu_tanh", lambda u: torch.nn.functional.gelu(u, approximate="tanh")),
                    ("gelu_erf", torch.nn.functional.gelu)):
        ops.gemm_simt(a, w, bias, out=out, act=act)
        assert float((out.double() - fn(ref)).abs().max()) < tol
    res = _rand(M, N, seed=10)
    res0 = res.clone()
    ops.gemm_simt(a, w, bias, residual=res)
    assert float((res.double() - (res0.double() + ref)).abs().max()) < tol
    # a row's result does not depend on the rows beside it
    if M > 1:
        one = torch.empty(1, N, device=DEV)
        ops.gemm_simt(a[M - 1:M], w, bias, out=one)
        ops.gemm_simt(a, w, bias, out=out)
        assert torch.equal(one[0], out[M - 1])
    # strided input rows (a column slice of a wider buffer)
    wide = _rand(M, K + 24, dtype=in_dtype, seed=11)
    ops.gemm_simt(wide[:, 8:8 + K], w, None, out=out)
    assert float((out.double() - wide[:, 8:8 + K].double() @ w.double().t()).abs().max()) < tol


def test_gemm_simt_same_bits_at_every_row_count():
    """The 32-bit product has a kernel for few rows, one for many rows and many features, and one
    between; a row's outputs have the same bits from each of them (one accumulator per output,
    k ascending), so that a token's logits do not depend on how many tokens its step brought."""
    ops = _ops()
    N, K = 1571, 772
    a, w, bias = _rand(1400, K, seed=21), _rand(N, K, seed=22, scale=0.1), _rand(N, seed=23)
    whole = torch.empty(1400, N, device=DEV)
    ops.gemm_simt(a, w, bias, out=whole, act="gelu_tanh")        # 128 x 128 blocks
    for lo, n in ((0, 1), (3, 8), (1384, 16), (100, 17), (640, 64), (700, 65), (0, 700)):
        part = torch.empty(n, N, device=DEV)
        ops.gemm_simt(a[lo:lo + n], w, bias, out=part, act="gelu_tanh")
        assert torch.equal(part, whole[lo:lo + n]), (lo, n)


def _paged_case(lens, q_lens, H, Hkv, D, page_size, dtype, seed, n_pages_extra=3, far_key=None):
    """Random requests laid out in shuffled pages.  Returns the kernel inputs and
    per-request dense K, V, and queries for the reference."""
    g = torch.Generator().manual_seed(seed)
    R = len(lens)
    n_blocks = [(n + page_size - 1) // page_size for n in lens]
    n_pages = sum(n_blocks) + n_pages_extra
    perm = torch.randperm(n_pages, generator=g).tolist()
    maxb = max(n_blocks) + 1
    bt = torch.full((R, maxb), -1, dtype=torch.int32)
    cache = torch.randn(n_pages, 2, Hkv, page_size, D, generator=g).to(dtype)   # garbage where unused
    Ks, Vs, Qs = [], [], []
    token_req, positions = [], []
    pi = 0
    for r, n in enumerate(lens):
        K = torch.randn(n, Hkv, D, generator=g)
        V = torch.randn(n, Hkv, D, generator=g)
        Q = torch.randn(q_lens[r], H, D, generator=g)
        if far_key is not None and n > far_key:
            # one far key stands out for the last query: the score at that key dominates
            K[far_key] = K[far_key] * 0 + Q[-1, ::H // Hkv][:Hkv] * 4.0
        K, V, Q = K.to(dtype), V.to(dtype), Q.to(dtype)
        for b in range(n_blocks[r]):
            page = perm[pi]
            pi += 1
            bt[r, b] = page
            lo, hi = b * page_size, min(n, (b + 1) * page_size)
            cache[page, 0, :, :hi - lo] = K[lo:hi].transpose(0, 1)
            cache[page, 1, :, :hi - lo] = V[lo:hi].transpose(0, 1)
        Ks.append(K)
        Vs.append(V)
        Qs.append(Q)
        for j in range(q_lens[r]):
            token_req.append(r)
            positions.append(n - q_lens[r] + j)
    q = torch.cat([x.reshape(x.shape[0], H * D) for x in Qs])
    return dict(q=q.to(DEV), cache=cache.to(DEV), bt=bt.to(DEV),
                token_req=torch.tensor(token_req, dtype=torch.int32, device=DEV),
                positions=torch.tensor(positions, dtype=torch.int32, device=DEV),
                Ks=Ks, Vs=Vs, Qs=Qs, lens=lens, q_lens=q_lens)


def _attention_reference(case, H, Hkv, D, scale, window):
    outs = []
    for K, V, Q, n, ql in zip(case["Ks"], case["Vs"], case["Qs"], case["lens"], case["q_lens"]):
        K, V, Q = K.double(), V.double(), Q.double()
        o = torch.zeros(ql, H, D, dtype=torch.float64)
        for j in range(ql):
            pos = n - ql + j
            lo = 0 if not window else max(0, pos - window + 1)
            for h in range(H):
                hk = h // (H // Hkv)
                s = (K[lo:pos + 1, hk] @ Q[j, h]) * scale
                w = torch.softmax(s, 0)
                o[j, h] = w @ V[lo:pos + 1, hk]
        outs.append(o.reshape(ql, H * D))
    return torch.cat(outs)


ATTN_CASES = [
    # lens, q_lens, H, Hkv, D, page_size, window
    ([1], [1], 1, 1, 16, 16, None),
    ([37, 5, 64], [37, 1, 3], 4, 4, 16, 16, None),
    ([100, 33], [2, 33], 3, 3, 32, 8, None),
    ([70, 129, 16], [1, 1, 1], 6, 2, 48, 16, None),        # grouped heads, head size 48
    ([65, 40], [65, 7], 5, 1, 80, 4, None),                # one key/value head for five query heads
    ([90, 50, 17], [30, 50, 1], 2, 2, 64, 16, 24),         # a window: its edge falls inside a page
    ([200], [200], 2, 1, 128, 32, 33),
    ([300, 9], [1, 9], 25, 25, 64, 16, None),              # 25 heads
]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("case_id", range(len(ATTN_CASES)))
def test_attention_simt_and_kv_write(case_id, dtype):
    ops = _ops()
    lens, q_lens, H, Hkv, D, ps, window = ATTN_CASES[case_id]
    c = _paged_case(lens, q_lens, H, Hkv, D, ps, dtype, seed=case_id)
    scale = 0.7 / math.sqrt(D)
    T = c["q"].shape[0]
    out = torch.empty(T, H * D, dtype=dtype, device=DEV)
    ops.attention_simt(c["q"], c["cache"], c["bt"], c["token_req"], c["positions"], out, H, scale,
                       window, max(lens))
    ref = _attention_reference(c, H, Hkv, D, scale, window)
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    assert float((out.double().cpu() - ref).abs().max()) < tol
    # kv_write puts the step's own keys and values where attention reads them
    cache2 = torch.zeros_like(c["cache"])
    for r, (K, V, n) in enumerate(zip(c["Ks"], c["Vs"], lens)):
        k_src = K.reshape(n, Hkv * D).to(DEV)
        v_src = V.reshape(n, Hkv * D).to(DEV)
        p = torch.arange(n)
        slots = (c["bt"][r].cpu()[p // ps].long() * ps + p % ps).to(torch.int32).to(DEV)
        ops.kv_write(k_src, v_src, cache2, slots, Hkv, D)
    out2 = torch.empty_like(out)
    ops.attention_simt(c["q"], cache2, c["bt"], c["token_req"], c["positions"], out2, H, scale,
                       window, max(lens))
    assert torch.equal(out2, out)


@pytest.mark.parametrize("M,H,Hkv,D,K,ps", [(300, 4, 4, 64, 256, 16), (1000, 8, 2, 128, 512, 16), (129, 2, 2, 32, 64, 8),
                                            (2048, 12, 12, 64, 768, 16),
                                            # queries that end inside a tile (192 and 1600 columns), one block a tile
                                            (300, 3, 3, 64, 256, 16), (300, 25, 25, 64, 1600, 16),
                                            # sizes that take the pair of blocks on a 256 x 256 tile: queries that
                                            # end inside a tile, and on a tile's edge
                                            (2048, 25, 25, 64, 1600, 16), (2000, 16, 16, 128, 2048, 32)])
def test_gemm_tc_kv_writes_what_projection_and_cache_write_would(M, H, Hkv, D, K, ps):
    """The query/key/value projection with the cache write in its epilogue: the same queries in
    `out`, the same bits in the same places of the cache as the plain product followed by
    kv_write; the key and value columns of `out` are not written; other pages are not touched."""
    ops = _ops()
    N = (H + 2 * Hkv) * D
    a, w, bias = _rand(M, K, dtype=torch.bfloat16, seed=31), _rand(N, K, dtype=torch.bfloat16, seed=32, scale=0.1), \
        _rand(N, seed=33)
    n_pages = (M + ps - 1) // ps + 5
    g = torch.Generator().manual_seed(M)
    slots = torch.randperm(n_pages * ps, generator=g)[:M].to(torch.int32).to(DEV)      # scattered over the pool
    plain = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    ops.gemm_tc(a, w, bias, out=plain)
    want = torch.full((n_pages, 2, Hkv, ps, D), 7.0, dtype=torch.bfloat16, device=DEV)
    ops.kv_write(plain[:, H * D:(H + Hkv) * D], plain[:, (H + Hkv) * D:], want, slots, Hkv, D)
    out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=DEV)
    cache = torch.full_like(want, 7.0)
    assert ops.gemm_tc_kv(a, w, bias, out, cache, slots, H, Hkv, D)
    assert torch.equal(out[:, :H * D], plain[:, :H * D])
    assert bool(torch.isnan(out[:, H * D:]).all())
    assert torch.equal(cache, want)


def test_gemm_tc_kv_declines_what_it_cannot_do():
    ops = _ops()
    for M, H, Hkv, D, K in ((64, 4, 4, 64, 256), (300, 4, 4, 48, 256), (300, 3, 3, 32, 256)):
        # few tokens (the other orientation); heads that are no multiple of 32 wide; queries that
        # do not end on a 64-column box (3 x 32 columns)
        N = (H + 2 * Hkv) * D
        a, w = _rand(M, K, dtype=torch.bfloat16, seed=1), _rand(N, K, dtype=torch.bfloat16, seed=2)
        out = torch.zeros(M, N, dtype=torch.bfloat16, device=DEV)
        cache = torch.zeros(M // 16 + 2, 2, Hkv, 16, D, dtype=torch.bfloat16, device=DEV)
        slots = torch.arange(M, dtype=torch.int32, device=DEV)
        done = ops.gemm_tc_kv(a, w, None, out, cache, slots, H, Hkv, D)
        if done:                       # (the third case may fall on 64-wide tiles)
            plain = torch.empty_like(out)
            ops.gemm_tc(a, w, None, out=plain)
            assert torch.equal(out[:, :H * D], plain[:, :H * D])
        else:
            assert float(out.abs().max()) == 0.0 and float(cache.abs().max()) == 0.0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_finds_a_far_key(dtype):
    """One key hundreds of positions back carries nearly all the weight: a kernel
    that loses it (a page's edge, a wrong block) is far off."""
    ops = _ops()
    H, Hkv, D, ps = 2, 2, 64, 16
    for far in (0, 15, 16, 255, 256, 300):
        c = _paged_case([700], [1], H, Hkv, D, ps, dtype, seed=far, far_key=far)
        out = torch.empty(1, H * D, dtype=dtype, device=DEV)
        ops.attention_simt(c["q"], c["cache"], c["bt"], c["token_req"], c["positions"], out, H, 1.0, None, 700)
        ref = _attention_reference(c, H, Hkv, D, 1.0, None)
        v_far = c["Vs"][0][far].double().reshape(-1)
        assert float((ref[0] - v_far).abs().max()) < 0.05        # the case is what it claims
        assert float((out.double().cpu() - ref).abs().max()) < (2e-5 if dtype == torch.float32 else 2e-2)


def _sampling_reference(row, p, u):
    """The kept set by thresholds (ties kept) and the draw in index order, float64."""
    l = row.astype(np.float64)
    if p["temperature"] <= 0:
        return int(np.argmax(l)), None
    w = np.exp((l - l.max()) / p["temperature"])
    S = w.sum()
    keep = np.ones_like(w, dtype=bool)
    if 0 < p["min_p"] < 1:
        keep &= w >= p["min_p"]
    if 0 < p["top_k"] < len(w):
        kept = np.sort(w[keep])[::-1]
        if len(kept) >= p["top_k"]:
            keep &= w >= kept[p["top_k"] - 1]
    if 0 < p["top_p"] < 1:
        order = np.argsort(-np.where(keep, w, -1), kind="stable")
        cum = np.cumsum(np.where(keep[order], w[order], 0.0))
        idx = np.searchsorted(cum, p["top_p"] * S, side="left")
        if idx < keep.sum():
            keep &= w >= w[order[idx]]
    cdf = np.cumsum(np.where(keep, w, 0.0))
    cdf /= cdf[-1]
    return keep, cdf


@pytest.mark.parametrize("V", [50, 1000, 50257])
def test_sampling(V):
    from sglang_c_b200.sampling import Sampler, SamplingParams
    g = torch.Generator().manual_seed(V)
    n = 12
    logits = (torch.randn(n, V, generator=g) * 2.0)
    logits[0, 7] = logits[0].max() + 1.0
    logits[0, 3] = logits[0, 7]                  # equal maxima: the lowest index wins
    params = [SamplingParams(),                               # greedy
              SamplingParams(temperature=0.0, top_k=5),
              SamplingParams(temperature=0.8),
              SamplingParams(temperature=1.3),
              SamplingParams(temperature=0.8, top_k=5),
              SamplingParams(temperature=1.0, top_k=1),
              SamplingParams(temperature=1.0, top_p=0.5),
              SamplingParams(temperature=0.7, top_p=0.9, top_k=20),
              SamplingParams(temperature=1.0, min_p=0.2),
              SamplingParams(temperature=0.8, top_k=50, top_p=0.95),   # the command line's defaults
              SamplingParams(temperature=1.0, top_k=10, top_p=0.3, min_p=0.05),
              SamplingParams(temperature=2.0, top_p=0.99)]
    s = Sampler(DEV, 16)
    rng = np.random.default_rng(V)
    for trial in range(6):
        us = [float(u) for u in rng.random(n)]
        if trial == 0:
            us = [0.0] * n
        if trial == 1:
            us = [0.9999999] * n
        dev = logits.clone().to(DEV)
        toks = s.sample(dev, params, us)
        for i in range(n):
            p = dict(temperature=params[i].temperature, top_k=params[i].top_k, top_p=params[i].top_p,
                     min_p=params[i].min_p)
            keep, cdf = _sampling_reference(logits[i].numpy(), p, us[i])
            if cdf is None:
                assert toks[i] == keep
                continue
            t = toks[i]
            assert keep[t], f"row {i}: token {t} is outside the kept set"
            lo = cdf[t - 1] if t > 0 else 0.0
            assert lo - 1e-4 <= us[i] <= cdf[t] + 1e-4, f"row {i}: u={us[i]} not in [{lo},{cdf[t]}]"
    assert toks[0] == 3


def test_sampling_penalties_and_logprob():
    from sglang_c_b200.sampling import Sampler, SamplingParams
    V = 300
    g = torch.Generator().manual_seed(1)
    logits = torch.randn(3, V, generator=g)
    top = int(logits[0].argmax())
    second = int(logits[0].topk(2).indices[1])
    logits[0, top] = abs(float(logits[0, top])) + 1.0
    s = Sampler(DEV, 8)
    params = [SamplingParams(repetition_penalty=100.0), SamplingParams(frequency_penalty=2.0, presence_penalty=0.5),
              SamplingParams()]
    hist = [[top, top], [int(logits[1].argmax())] * 3, [1, 2, 3]]
    dev = logits.clone().to(DEV)
    toks, lps = s.sample(dev, params, [0.0] * 3, histories=hist, want_logprobs=True)
    assert toks[0] == second
    l1 = logits[1].clone().double()
    l1[hist[1][0]] -= 2.0 * 3 + 0.5
    assert toks[1] == int(l1.argmax())
    assert abs(lps[1] - float(torch.log_softmax(l1, 0)[toks[1]])) < 1e-4
    assert toks[2] == int(logits[2].argmax())
    assert abs(lps[2] - float(torch.log_softmax(logits[2].double(), 0)[toks[2]])) < 1e-4


GEMM_TC_SHAPES = [
    # M, N, K: few tokens (weights on the MMA's 128-row side, split-K) and many tokens
    (1, 768, 768), (8, 2304, 768), (8, 768, 3072), (16, 3072, 768), (17, 100, 64), (64, 768, 768),
    (33, 1000, 96), (100, 320, 96), (128, 50257, 64), (3, 96, 320), (5, 777, 128), (128, 128, 128),
    (129, 768, 768), (300, 2304, 768), (2048, 768, 3072), (1000, 1000, 200), (257, 96, 320),
    (512, 50257 // 8, 96), (130, 72, 8), (2, 8, 8),
    (200, 128, 2048), (400, 200, 3000),      # few tiles and a long K; a K that ends inside a block of 64
    # sizes that take a pair of blocks on a 256 x 256 tile; the last with ragged rows, columns and K
    (2048, 6400, 1600), (2048, 1600, 6400), (1100, 3000, 1608),
]


def test_gemm_tc_shapes_reach_all_three_kernels():
    """The sizes above are chosen for a kernel each; the library says which one a size takes."""
    ops = _ops()
    forms = {(M, N, K): ops.gemm_tc_form(M, N, K) for M, N, K in GEMM_TC_SHAPES}
    assert forms[(8, 2304, 768)] == "few" and forms[(64, 768, 768)] == "few" and forms[(33, 1000, 96)] == "few"
    # (from 65 tokens on a product over a short K takes the many-token kernel)
    assert forms[(2048, 768, 3072)] == "stream" and forms[(129, 768, 768)] == "stream" and forms[(128, 50257, 64)] == "stream"
    for size in ((2048, 6400, 1600), (2048, 1600, 6400), (1100, 3000, 1608)):
        assert forms[size] == "pair"
    # and the projections of test_gemm_tc_kv_...: queries ending inside a tile, on one block and on a pair
    assert ops.gemm_tc_form(300, 3 * 25 * 64, 1600) == "stream" and ops.gemm_tc_form(2048, 3 * 25 * 64, 1600) == "pair"
    assert ops.gemm_tc_form(2000, 3 * 16 * 128, 2048) == "pair" and ops.gemm_tc_form(2048, 2304, 768) == "pair"


@pytest.mark.parametrize("M,N,K", GEMM_TC_SHAPES)
def test_gemm_tc(M, N, K):
    """The tcgen05 GEMM against a float64 product of the same bfloat16 operands."""
    ops = _ops()
    a, w, bias = _rand(M, K, dtype=torch.bfloat16, seed=20), _rand(N, K, dtype=torch.bfloat16, seed=21, scale=0.1), _rand(N, seed=22)
    assert ops.gemm_tc_supported(a, w)
    ref = a.double() @ w.double().t() + bias.double()
    tol32 = 2e-5 * math.sqrt(K) + 1e-5
    out = torch.full((M, N), float("nan"), device=DEV)
    ops.gemm_tc(a, w, bias, out=out)
    assert float((out.double() - ref).abs().max()) < tol32
    outb = torch.zeros(M, N, dtype=torch.bfloat16, device=DEV)
    ops.gemm_tc(a, w, bias, out=outb, act="gelu_tanh")
    want = torch.nn.functional.gelu(ref, approximate="tanh")
    assert float((outb.double() - want).abs().max()) < tol32 + 8e-3 * float(want.abs().max())
    ops.gemm_tc(a, w, None, out=outb, act="gelu_erf")
    want = torch.nn.functional.gelu(ref - bias.double())
    assert float((outb.double() - want).abs().max()) < tol32 + 8e-3 * float(want.abs().max())
    res = _rand(M, N, seed=23)
    res0 = res.clone()
    ops.gemm_tc(a, w, bias, residual=res)
    assert float((res.double() - (res0.double() + ref)).abs().max()) < tol32
    # the same call twice gives the same bits (the split-K sum has a fixed order)
    out2 = torch.empty(M, N, device=DEV)
    ops.gemm_tc(a, w, bias, out=out2)
    assert torch.equal(out, out2)
    # strided input rows and a wider output buffer
    wide = _rand(M, K + 16, dtype=torch.bfloat16, seed=24)
    big = torch.zeros(M, N + 5, device=DEV)
    if (K + 16) % 8 == 0:
        ops.gemm_tc(wide[:, 8:8 + K], w, None, out=big[:, :N])
        assert float((big[:, :N].double() - wide[:, 8:8 + K].double() @ w.double().t()).abs().max()) < tol32
        assert float(big[:, N:].abs().max()) == 0.0
    assert int(ops.tc_error_flag(a.device).item()) == 0


GEMM_FEW_SHAPES = [(1, 8, 8), (3, 13, 40), (8, 100, 72), (1, 768, 768), (2, 30, 1600), (5, 2304, 768),
                   (2, 768, 3072), (2, 65, 3080), (4, 17, 6400), (7, 1031, 96)]


@pytest.mark.parametrize("M,N,K", GEMM_FEW_SHAPES)
def test_gemm_few(M, N, K):
    """The few-token product (weights and tokens from global memory into the registers of the
    warp-level tensor-core instruction) against a float64 product of the same operands."""
    ops = _ops()
    a, w, bias = _rand(M, K, dtype=torch.bfloat16, seed=30), _rand(N, K, dtype=torch.bfloat16, seed=31, scale=0.1), _rand(N, seed=32)
    ref = a.double() @ w.double().t() + bias.double()
    tol32 = 2e-5 * math.sqrt(K) + 1e-5
    out = torch.full((M, N), float("nan"), device=DEV)
    ops.gemm_few(a, w, bias, out=out)
    assert float((out.double() - ref).abs().max()) < tol32
    outb = torch.zeros(M, N, dtype=torch.bfloat16, device=DEV)
    ops.gemm_few(a, w, bias, out=outb, act="gelu_tanh")
    want = torch.nn.functional.gelu(ref, approximate="tanh")
    assert float((outb.double() - want).abs().max()) < tol32 + 8e-3 * float(want.abs().max())
    ops.gemm_few(a, w, None, out=outb, act="gelu_erf")
    want = torch.nn.functional.gelu(ref - bias.double())
    assert float((outb.double() - want).abs().max()) < tol32 + 8e-3 * float(want.abs().max())
    res = _rand(M, N, seed=33)
    res0 = res.clone()
    ops.gemm_few(a, w, bias, residual=res)
    assert float((res.double() - (res0.double() + ref)).abs().max()) < tol32
    out2 = torch.empty(M, N, device=DEV)
    ops.gemm_few(a, w, bias, out=out2)
    assert torch.equal(out, out2)
    # strided input rows and a wider output buffer; rows of the buffer beyond M stay as they are
    wide = _rand(M, K + 16, dtype=torch.bfloat16, seed=34)
    big = torch.zeros(M + 2, N + 5, device=DEV)
    ops.gemm_few(wide[:, 8:8 + K], w, None, out=big[:, :N])
    assert float((big[:M, :N].double() - wide[:, 8:8 + K].double() @ w.double().t()).abs().max()) < tol32
    assert float(big[:, N:].abs().max()) == 0.0 and float(big[M:].abs().max()) == 0.0
    # the same product through the tcgen05 kernel agrees to rounding of the sum's order
    out3 = torch.empty(M, N, device=DEV)
    ops.gemm_tc(a, w, bias, out=out3)
    assert float((out3 - out).abs().max()) < tol32


def test_gemm_few_refuses_what_it_cannot_take():
    ops = _ops()
    w = _rand(6, 64, dtype=torch.bfloat16)
    with pytest.raises(ops.KernelError):
        ops.gemm_few(_rand(9, 64, dtype=torch.bfloat16), w, None, out=torch.empty(9, 6, device=DEV))
    with pytest.raises(ops.KernelError):
        ops.gemm_few(_rand(4, 100, dtype=torch.bfloat16), _rand(6, 100, dtype=torch.bfloat16), None,
                     out=torch.empty(4, 6, device=DEV))


def test_gemm_tc_refuses_rows_that_tma_cannot_load():
    ops = _ops()
    a, w = _rand(4, 100, dtype=torch.bfloat16), _rand(6, 100, dtype=torch.bfloat16)
    assert not ops.gemm_tc_supported(a, w)            # K = 100 is not a multiple of 8
    with pytest.raises(ops.KernelError):
        ops.gemm_tc(a, w, None, out=torch.empty(4, 6, device=DEV))


@pytest.mark.parametrize("case_id", range(len(ATTN_CASES)))
@pytest.mark.parametrize("tokens", ["last", "all"])
def test_attention_decode(case_id, tokens):
    """The split-key decode kernel: one query per request ("last"), and the same kernel given
    every token of a portion ("all": each token is an independent query)."""
    ops = _ops()
    lens, q_lens, H, Hkv, D, ps, window = ATTN_CASES[case_id]
    if tokens == "last":
        q_lens = [1] * len(lens)
    c = _paged_case(lens, q_lens, H, Hkv, D, ps, torch.bfloat16, seed=100 + case_id)
    scale = 0.9 / math.sqrt(D)
    T = c["q"].shape[0]
    ref = _attention_reference(c, H, Hkv, D, scale, window)
    for max_keys in (max(lens), 1024):          # 1024: as under a captured graph
        out = torch.full((T, H * D), float("nan"), dtype=torch.bfloat16, device=DEV)
        ops.attention_decode(c["q"], c["cache"], c["bt"], c["token_req"], c["positions"], out, H, scale,
                             window, max_keys)
        assert float((out.double().cpu() - ref).abs().max()) < 2e-2
        out2 = torch.empty_like(out)
        ops.attention_decode(c["q"], c["cache"], c["bt"], c["token_req"], c["positions"], out2, H, scale,
                             window, max_keys)
        assert torch.equal(out, out2)             # fixed merge order


def test_attention_decode_finds_a_far_key():
    ops = _ops()
    H, Hkv, D, ps = 2, 2, 64, 16
    for far in (0, 15, 16, 63, 64, 255, 256, 300, 699):
        c = _paged_case([700], [1], H, Hkv, D, ps, torch.bfloat16, seed=far, far_key=far)
        out = torch.empty(1, H * D, dtype=torch.bfloat16, device=DEV)
        ops.attention_decode(c["q"], c["cache"], c["bt"], c["token_req"], c["positions"], out, H, 1.0, None, 700)
        ref = _attention_reference(c, H, Hkv, D, 1.0, None)
        assert float((out.double().cpu() - ref).abs().max()) < 2e-2, far


PREFILL_TC_CASES = [
    # lens, q_lens, H, Hkv, D, page_size, window
    ([1], [1], 1, 1, 64, 16, None),
    ([37, 5, 64], [37, 1, 3], 3, 3, 64, 16, None),
    ([128, 129, 127], [128, 129, 127], 2, 2, 64, 16, None),        # tile edges
    ([300, 200], [44, 200], 4, 2, 64, 8, None),                    # a portion after 256 cached keys
    ([1000], [1000], 2, 1, 64, 16, None),
    ([260, 90], [260, 1], 2, 2, 128, 16, None),                    # head size 128
    ([500, 70], [300, 70], 2, 2, 64, 16, 100),                     # a window that ends inside a tile
    ([400], [400], 1, 1, 128, 32, 129),
    ([700, 3, 130], [2, 3, 130], 12, 12, 64, 16, None),
    ([900], [900], 2, 1, 128, 16, None),                           # head size 128, query tiles shared by two blocks
    ([1100], [1100], 1, 1, 64, 16, 800),                           # shared tiles whose first key tile meets the window
    ([1500, 40], [700, 40], 2, 2, 64, 32, None),                   # a portion after 800 cached keys: 7 to 12 key tiles
    ([300, 129, 900], [300, 20, 900], 2, 2, 64, 48, None),         # pages that do not divide a tile: loads by cp.async
    ([200], [200], 1, 1, 128, 24, 150),
]


@pytest.mark.parametrize("case_id", range(len(PREFILL_TC_CASES)))
def test_attention_prefill_tc(case_id):
    ops = _ops()
    lens, q_lens, H, Hkv, D, ps, window = PREFILL_TC_CASES[case_id]
    c = _paged_case(lens, q_lens, H, Hkv, D, ps, torch.bfloat16, seed=200 + case_id)
    scale = 1.1 / math.sqrt(D)
    T = c["q"].shape[0]
    q_start = torch.tensor([0] + list(np.cumsum(q_lens)), dtype=torch.int32, device=DEV)
    kv_len = torch.tensor(lens, dtype=torch.int32, device=DEV)
    out = torch.full((T, H * D), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.attention_prefill_tc(c["q"], c["cache"], c["bt"], q_start, kv_len, out, H, scale, window,
                             len(lens), max(q_lens))
    ref = _attention_reference(c, H, Hkv, D, scale, window)
    err = float((out.double().cpu() - ref).abs().max())
    assert err < 2e-2, err
    assert int(ops.tc_error_flag(out.device).item()) == 0
    # the plain kernel on the same inputs agrees too
    out2 = torch.empty_like(out)
    ops.attention_simt(c["q"], c["cache"], c["bt"], c["token_req"], c["positions"], out2, H, scale, window, max(lens))
    assert float((out.float() - out2.float()).abs().max()) < 2e-2


def test_attention_prefill_tc_finds_a_far_key():
    ops = _ops()
    H, Hkv, D, ps = 2, 2, 64, 16
    for far in (0, 127, 128, 255, 300, 511, 512, 699):
        c = _paged_case([700], [130], H, Hkv, D, ps, torch.bfloat16, seed=far, far_key=far if far < 570 else 569)
        q_start = torch.tensor([0, 130], dtype=torch.int32, device=DEV)
        kv_len = torch.tensor([700], dtype=torch.int32, device=DEV)
        out = torch.empty(130, H * D, dtype=torch.bfloat16, device=DEV)
        ops.attention_prefill_tc(c["q"], c["cache"], c["bt"], q_start, kv_len, out, H, 1.0, None, 1, 130)
        ref = _attention_reference(c, H, Hkv, D, 1.0, None)
        assert float((out.double().cpu() - ref).abs().max()) < 3e-2, far


@pytest.mark.parametrize("case_id", [1, 3, 4, 7])
def test_attention_decode_writes_new_keys_itself(case_id):
    """One token per request: the kernel takes the token's own key and value from the step's
    rows and writes them into the cache; afterwards the cache holds what kv_write would have put."""
    ops = _ops()
    lens, _, H, Hkv, D, ps, window = ATTN_CASES[case_id]
    c = _paged_case(lens, [1] * len(lens), H, Hkv, D, ps, torch.bfloat16, seed=300 + case_id)
    scale = 1.0 / math.sqrt(D)
    T = len(lens)
    ref = _attention_reference(c, H, Hkv, D, scale, window)
    k_new = torch.stack([K[-1].reshape(-1) for K in c["Ks"]]).to(DEV)
    v_new = torch.stack([V[-1].reshape(-1) for V in c["Vs"]]).to(DEV)
    slots = torch.tensor([int(c["bt"][r, (n - 1) // ps]) * ps + (n - 1) % ps for r, n in enumerate(lens)],
                         dtype=torch.int32, device=DEV)
    want_cache = c["cache"].clone()
    holed = c["cache"].clone()
    for r, n in enumerate(lens):                      # the last position is not in the cache yet
        holed[int(c["bt"][r, (n - 1) // ps]), :, :, (n - 1) % ps] = 7.0
    out = torch.empty(T, H * D, dtype=torch.bfloat16, device=DEV)
    ops.attention_decode(c["q"], holed, c["bt"], c["token_req"], c["positions"], out, H, scale, window,
                         max(lens), k_new=k_new, v_new=v_new, slots=slots)
    assert float((out.double().cpu() - ref).abs().max()) < 2e-2
    assert torch.equal(holed, want_cache)


def test_attention_kernels_share_a_mixed_step():
    """Portions of some requests beside single tokens of others: the tile kernel serves the
    portions and skips the single tokens, the split-key kernel serves exactly those."""
    ops = _ops()
    lens, q_lens, H, Hkv, D, ps = [300, 200, 77, 513, 64], [44, 1, 1, 130, 1], 4, 2, 64, 16
    c = _paged_case(lens, q_lens, H, Hkv, D, ps, torch.bfloat16, seed=900)
    scale = 1.0 / math.sqrt(D)
    T = c["q"].shape[0]
    q_start = torch.tensor([0] + list(np.cumsum(q_lens)), dtype=torch.int32, device=DEV)
    kv_len = torch.tensor(lens, dtype=torch.int32, device=DEV)
    singles = [int(q_start[r]) for r, n in enumerate(q_lens) if n == 1]
    token_list = torch.tensor(singles + [0, 0], dtype=torch.int32, device=DEV)
    out = torch.full((T, H * D), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.attention_prefill_tc(c["q"], c["cache"], c["bt"], q_start, kv_len, out, H, scale, None, len(lens),
                             max(q_lens), skip_single=True)
    torch.cuda.synchronize()
    assert all(bool(torch.isnan(out[t]).all()) for t in singles)          # left for the other kernel
    ops.attention_decode(c["q"], c["cache"], c["bt"], c["token_req"], c["positions"], out, H, scale, None,
                         max(lens), token_list=token_list, n_tokens=len(singles))
    ref = _attention_reference(c, H, Hkv, D, scale, None)
    assert float((out.double().cpu() - ref).abs().max()) < 2e-2


STREAM_CASES = [
    # lens, H, Hkv, D, page_size, window
    ([1, 2, 17, 64, 65, 300], 3, 3, 64, 16, None),
    ([700, 3, 130, 64], 12, 12, 64, 16, None),
    ([90, 50, 17, 200], 2, 2, 64, 16, 24),                 # a window: its edge falls inside a page
    ([300, 129], 6, 2, 64, 8, None),                       # grouped heads, small pages
    ([260, 90, 1], 2, 2, 128, 16, None),                   # head size 128
    ([200, 77], 2, 1, 128, 32, 33),
    ([500, 64, 63], 4, 4, 64, 64, None),                   # a page per stage
    ([130, 9], 5, 5, 64, 8, 100),
    (list(range(1, 61)), 12, 12, 64, 16, None),            # 720 items: blocks walk several items each
    ([1500] + [40] * 50, 10, 10, 64, 16, None),            # one long request among short ones
    ([1100] * 40, 12, 12, 64, 16, None),                   # several long items per block
    ([77, 200, 3], 3, 1, 128, 64, None),                   # head size 128, a page per stage
]


@pytest.mark.parametrize("case_id", range(len(STREAM_CASES)))
def test_attention_decode_streaming_kernel(case_id):
    """The streaming decode kernel (resident blocks walking (token, head) items through a ring of
    TMA stages) against the float64 reference; rows of the cache that hold no key are NaN, so a
    masked row that leaked into a sum would show.  Also with the token's own key and value taken
    from the step's rows and written into the cache by the kernel."""
    ops = _ops()
    lens, H, Hkv, D, ps, window = STREAM_CASES[case_id]
    c = _paged_case(lens, [1] * len(lens), H, Hkv, D, ps, torch.bfloat16, seed=500 + case_id)
    scale = 1.0 / math.sqrt(D)
    T = len(lens)
    ref = _attention_reference(c, H, Hkv, D, scale, window)
    used = torch.zeros(c["cache"].shape[0], ps, dtype=torch.bool)
    for r, n in enumerate(lens):
        for p in range(n):
            used[int(c["bt"][r, p // ps]), p % ps] = True
    cache = c["cache"].clone()
    cache[(~used).to(DEV)[:, None, None, :].expand(-1, 2, Hkv, -1)] = float("nan")
    for max_keys in (max(lens), max(1024, max(lens))):
        out = torch.full((T, H * D), float("nan"), dtype=torch.bfloat16, device=DEV)
        ops.attention_decode(c["q"], cache, c["bt"], c["token_req"], c["positions"], out, H, scale, window,
                             max_keys, variant="stream")
        err = float((out.double().cpu() - ref).abs().max())
        assert err < 2e-2, err
        out2 = torch.empty_like(out)
        ops.attention_decode(c["q"], cache, c["bt"], c["token_req"], c["positions"], out2, H, scale, window,
                             max_keys, variant="stream")
        assert torch.equal(out, out2)
    # the token's own key and value from the step's rows; its cache row is not written yet
    k_new = torch.stack([K[-1].reshape(-1) for K in c["Ks"]]).to(DEV)
    v_new = torch.stack([V[-1].reshape(-1) for V in c["Vs"]]).to(DEV)
    slots = torch.tensor([int(c["bt"][r, (n - 1) // ps]) * ps + (n - 1) % ps for r, n in enumerate(lens)],
                         dtype=torch.int32, device=DEV)
    holed = cache.clone()
    for r, n in enumerate(lens):
        holed[int(c["bt"][r, (n - 1) // ps]), :, :, (n - 1) % ps] = float("nan")
    out3 = torch.full((T, H * D), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.attention_decode(c["q"], holed, c["bt"], None if case_id % 2 else c["token_req"], c["positions"], out3, H,
                         scale, window, max(lens), k_new=k_new, v_new=v_new, slots=slots, variant="stream")
    assert torch.equal(out3, out)
    assert torch.equal(torch.nan_to_num(holed, nan=-7.0), torch.nan_to_num(cache, nan=-7.0))
    # all tokens in an order (long contexts first, as the engine lists them): the same result
    order = torch.tensor(sorted(range(T), key=lambda t: -lens[t]), dtype=torch.int32, device=DEV)
    for fused in (False, True):
        holed2 = cache.clone()
        if fused:
            for r, n in enumerate(lens):
                holed2[int(c["bt"][r, (n - 1) // ps]), :, :, (n - 1) % ps] = float("nan")
        out4 = torch.full((T, H * D), float("nan"), dtype=torch.bfloat16, device=DEV)
        ops.attention_decode(c["q"], holed2, c["bt"], c["token_req"] if case_id % 2 else None, c["positions"], out4,
                             H, scale, window, max(lens), k_new=k_new if fused else None,
                             v_new=v_new if fused else None, slots=slots if fused else None,
                             token_list=order, n_tokens=T, variant="stream")
        assert torch.equal(out4, out), fused
        assert torch.equal(torch.nan_to_num(holed2, nan=-7.0), torch.nan_to_num(cache, nan=-7.0))
    assert int(ops.tc_error_flag(out.device).item()) == 0


def test_attention_decode_streaming_kernel_finds_a_far_key_and_serves_a_token_list():
    ops = _ops()
    H, Hkv, D, ps = 2, 2, 64, 16
    for far in (0, 15, 16, 63, 64, 255, 256, 300, 698):
        c = _paged_case([700], [1], H, Hkv, D, ps, torch.bfloat16, seed=far, far_key=far)
        out = torch.empty(1, H * D, dtype=torch.bfloat16, device=DEV)
        ops.attention_decode(c["q"], c["cache"], c["bt"], c["token_req"], c["positions"], out, H, 1.0, None, 700,
                             variant="stream")
        ref = _attention_reference(c, H, Hkv, D, 1.0, None)
        assert float((out.double().cpu() - ref).abs().max()) < 2e-2, far
    # single tokens picked out of a mixed step by a list
    lens, q_lens, H, Hkv = [300, 200, 77, 513, 64], [44, 1, 1, 130, 1], 4, 2
    c = _paged_case(lens, q_lens, H, Hkv, D, ps, torch.bfloat16, seed=901)
    q_start = [0] + list(np.cumsum(q_lens))
    singles = [int(q_start[r]) for r, n in enumerate(q_lens) if n == 1]
    token_list = torch.tensor(singles + [0, 0], dtype=torch.int32, device=DEV)
    T = c["q"].shape[0]
    out = torch.full((T, H * D), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.attention_decode(c["q"], c["cache"], c["bt"], c["token_req"], c["positions"], out, H, 0.125, None,
                         max(lens), token_list=token_list, n_tokens=len(singles), variant="stream")
    ref = _attention_reference(c, H, Hkv, D, 0.125, None)
    got = out.double().cpu()
    for t in range(T):
        if t in singles:
            assert float((got[t] - ref[t]).abs().max()) < 2e-2
        else:
            assert bool(torch.isnan(out[t]).all())


def test_both_decode_attention_kernels_at_head_size_64():
    """Head sizes 64 and 128 go to the TMA-staged kernel by default; the register-staged one
    must give the same there (it serves the other head sizes and more than 8 key ranges)."""
    ops = _ops()
    for case_id in (5, 6, 7):
        lens, _, H, Hkv, D, ps, window = ATTN_CASES[case_id]
        c = _paged_case(lens, [1] * len(lens), H, Hkv, D, ps, torch.bfloat16, seed=400 + case_id)
        scale = 1.0 / math.sqrt(D)
        ref = _attention_reference(c, H, Hkv, D, scale, window)
        outs = []
        for use_tma in (True, False):
            ops.USE_TMA_DECODE = use_tma
            try:
                out = torch.full((len(lens), H * D), float("nan"), dtype=torch.bfloat16, device=DEV)
                ops.attention_decode(c["q"], c["cache"], c["bt"], c["token_req"], c["positions"], out, H, scale,
                                     window, max(lens))
            finally:
                ops.USE_TMA_DECODE = True
            assert float((out.double().cpu() - ref).abs().max()) < 2e-2, (case_id, use_tma)
            outs.append(out)
        assert float((outs[0].float() - outs[1].float()).abs().max()) < 1e-2
