"""Each CUDA kernel alone against its plain PyTorch restatement
(tests/reference_ops.py), at sizes other than the engine tests use: head sizes
16/48/128, group sizes 1/2/5, widths and vocabularies that are no power of two,
token counts that are no multiple of a tile, positions that straddle pages."""
import math

import pytest
import torch

from reference_ops import ReferenceKernels

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


@pytest.fixture(scope="module")
def k():
    from chibillm_b200.kernels.ops import CudaKernels
    return CudaKernels(torch.device("cuda:0"))


@pytest.fixture(scope="module")
def ref():
    return ReferenceKernels()


def rnd(*shape, dtype=torch.float32, seed=0, scale=1.0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(*shape, generator=g, device="cuda") * scale).to(dtype)


def close(a, b, dtype, what, rel=None):
    a, b = a.float(), b.float()
    scale = float(b.abs().max()) + 1e-30
    tol = rel if rel is not None else (3e-6 if dtype == torch.float32 else 1.2e-2)
    worst = float((a - b).abs().max())
    assert torch.isfinite(a).all(), f"{what}: not finite"
    assert worst <= tol * scale, f"{what}: max |diff| {worst:.3e} > {tol:.1e} * {scale:.3e}"


@pytest.mark.parametrize("wdtype", DTYPES)
def test_embed(k, ref, wdtype):
    table = rnd(1000, 200, dtype=wdtype)
    tokens = torch.tensor([0, 999, 5, 5, 731], dtype=torch.int32, device="cuda")
    out = torch.full((5, 200), float("nan"), device="cuda")
    exp = torch.empty_like(out)
    k.embed(tokens, table, out)
    ref.embed(tokens, table, exp)
    assert torch.equal(out, exp)


@pytest.mark.parametrize("n", [16, 200, 4096])
@pytest.mark.parametrize("xdtype,odtype", [(torch.float32, torch.float32), (torch.float32, torch.bfloat16),
                                           (torch.bfloat16, torch.bfloat16)])
def test_rmsnorm(k, ref, n, xdtype, odtype):
    x = rnd(37, n, dtype=xdtype, seed=1, scale=3.0)
    w = (1 + 0.1 * rnd(n, seed=2)).to(odtype)
    out = torch.full((37, n), float("nan"), dtype=odtype, device="cuda")
    exp = torch.empty_like(out)
    k.rmsnorm(x, w, 1e-5, 0.0, out)
    ref.rmsnorm(x, w, 1e-5, 0.0, exp)
    close(out, exp, odtype, "rmsnorm", rel=3e-6 if odtype == torch.float32 else 8e-3)
    # strided rows and a weight offset
    wide = rnd(9, 3 * n, dtype=xdtype, seed=3)
    view = wide[:, n:2 * n]
    out2 = torch.empty(9, n, dtype=odtype, device="cuda")
    exp2 = torch.empty_like(out2)
    k.rmsnorm(view, w, 1e-6, 1.0, out2)
    ref.rmsnorm(view, w, 1e-6, 1.0, exp2)
    close(out2, exp2, odtype, "rmsnorm strided", rel=3e-6 if odtype == torch.float32 else 8e-3)


@pytest.mark.parametrize("M", [1, 5, 64, 130])
@pytest.mark.parametrize("xdtype,wdtype,odtype", [
    (torch.float32, torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16, torch.bfloat16),
    (torch.bfloat16, torch.bfloat16, torch.float32), (torch.float32, torch.bfloat16, torch.float32),
    (torch.bfloat16, torch.float32, torch.bfloat16)])
def test_linear(k, ref, M, xdtype, wdtype, odtype):
    N, K = 203, 100
    x = rnd(M, K, dtype=xdtype, seed=4)
    w = rnd(N, K, dtype=wdtype, seed=5, scale=0.1)
    out = torch.full((M, N), float("nan"), dtype=odtype, device="cuda")
    exp = torch.empty_like(out)
    k.linear(x, w, out)
    ref.linear(x, w, exp)
    close(out, exp, odtype, "linear")
    if odtype == torch.float32:
        res = rnd(M, N, seed=6)
        exp_res = torch.empty_like(res)
        ref.linear(x, w, exp_res, residual=res)
        k.linear(x, w, res, residual=res)          # in place
        close(res, exp_res, odtype, "linear + residual")


def _paged_setup(seq_ctx, q_lens, page_size, num_pages, seed):
    """Block tables through shuffled pages for sequences that hold ``seq_ctx``
    tokens after feeding their last ``q_lens`` ones."""
    g = torch.Generator().manual_seed(seed)
    perm = torch.randperm(num_pages, generator=g).tolist()
    S = len(seq_ctx)
    width = max((c + page_size - 1) // page_size for c in seq_ctx)
    table = torch.full((S, width), -1, dtype=torch.int32)
    cursor = 0
    for s, c in enumerate(seq_ctx):
        n = (c + page_size - 1) // page_size
        table[s, :n] = torch.tensor(perm[cursor:cursor + n], dtype=torch.int32)
        cursor += n
    assert cursor <= num_pages
    positions, seq_of_token, q_start = [], [], [0]
    for s, (c, n) in enumerate(zip(seq_ctx, q_lens)):
        positions += list(range(c - n, c))
        seq_of_token += [s] * n
        q_start.append(q_start[-1] + n)
    dev = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")
    return table.cuda(), dev(positions), dev(seq_of_token), dev(q_start), dev(seq_ctx)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nq,nkv,d,rot,norms", [(6, 2, 48, 48, True), (4, 4, 16, 8, True),
                                                (5, 1, 128, 128, False), (2, 1, 32, 0, True),
                                                (9, 3, 128, 128, True)])
@pytest.mark.parametrize("seq_ctx,q_lens", [([19, 8, 70], [19, 1, 7]),
                                            ([70, 8, 90], [40, 1, 33])])   # many tokens: the per-token kernel
def test_qk_norm_rope_append(k, ref, dtype, nq, nkv, d, rot, norms, seq_ctx, q_lens):
    page, pages = 8, 40
    table, positions, seq_of_token, _, _ = _paged_setup(seq_ctx, q_lens, page, pages, seed=7)
    T = sum(q_lens)
    qkv = rnd(T, (nq + 2 * nkv) * d, dtype=dtype, seed=8)
    qn = (1 + 0.1 * rnd(d, seed=9)).to(dtype) if norms else None
    kn = (1 + 0.1 * rnd(d, seed=10)).to(dtype) if norms else None
    inv_freq = torch.pow(torch.tensor(1e4), -2 * torch.arange(max(rot, 2) // 2, dtype=torch.float32) / max(rot, 2)).cuda()
    outs = []
    for impl in (k, ref):
        q_out = torch.full((T, nq * d), float("nan"), dtype=dtype, device="cuda")
        kc = torch.full((pages, nkv, page, d), 7.0, dtype=dtype, device="cuda")
        vc = torch.full((pages, nkv, page, d), 7.0, dtype=dtype, device="cuda")
        impl.qk_norm_rope_append(qkv, q_out, kc, vc, qn, kn, inv_freq if rot else None, rot, 1e-6, 0.0,
                                 positions, seq_of_token, table, nq, nkv, d, page)
        outs.append((q_out, kc, vc))
    if hasattr(k, "check_error_word"):
        k.check_error_word()
    tol = 3e-6 if dtype == torch.float32 else 8e-3
    close(outs[0][0], outs[1][0], dtype, "q", rel=tol)
    close(outs[0][1], outs[1][1], dtype, "key cache", rel=tol)
    assert torch.equal(outs[0][2], outs[1][2]), "value cache"
    # q only: a layer that reads another layer's cache
    q_only = torch.empty(T, nq * d, dtype=dtype, device="cuda")
    k.qk_norm_rope_append(qkv[:, :nq * d].contiguous(), q_only, None, None, qn, kn,
                          inv_freq if rot else None, rot, 1e-6, 0.0, positions, seq_of_token, None,
                          nq, nkv, d, page)
    close(q_only, outs[1][0], dtype, "q only", rel=tol)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nq,nkv,d,window", [(4, 2, 16, None), (6, 3, 48, 24), (5, 1, 128, None),
                                             (8, 8, 64, 7), (10, 2, 32, 33), (20, 1, 64, None),
                                             (4, 1, 256, 100)])
@pytest.mark.parametrize("seq_ctx,q_lens", [
    # whole prompts, single decoded tokens at page edges, a portion in the middle
    ([33, 64, 65, 16, 150], [33, 1, 1, 16, 21]),
    # decoding only, contexts of very different lengths
    ([1, 17, 128, 129, 400], [1, 1, 1, 1, 1]),
    # portions only, one of them longer than a tile of query rows
    ([200, 90], [130, 2])])
def test_attention_against_plain(k, ref, dtype, nq, nkv, d, window, seq_ctx, q_lens):
    page, pages = 8, 128
    table, positions, seq_of_token, q_start, ctx_len = _paged_setup(seq_ctx, q_lens, page, pages, seed=11)
    T = sum(q_lens)
    q = rnd(T, nq * d, dtype=dtype, seed=12)
    # pages that no sequence owns hold NaN: reading one would show
    kc = torch.full((pages, nkv, page, d), float("nan"), dtype=dtype, device="cuda")
    vc = torch.full((pages, nkv, page, d), float("nan"), dtype=dtype, device="cuda")
    for s, c in enumerate(seq_ctx):
        idx = torch.arange(c, device="cuda")
        pg = table[s, idx // page].long()
        kc[pg, :, idx % page, :] = rnd(c, nkv, d, dtype=dtype, seed=1000 + s)
        vc[pg, :, idx % page, :] = rnd(c, nkv, d, dtype=dtype, seed=5000 + s)
    out = torch.full((T, nq * d), float("nan"), dtype=dtype, device="cuda")
    exp = torch.empty_like(out)
    scale = 1.0 / math.sqrt(d)
    args = (table, q_start, ctx_len, seq_of_token, positions, nq, nkv, d, page, scale, window,
            max(q_lens), max(seq_ctx), min(q_lens))
    k.attention(q, kc, vc, out, *args)
    ref.attention(q, kc, vc, exp, *args)
    k.check_error_word()
    close(out, exp, dtype, "attention", rel=1e-5 if dtype == torch.float32 else 1.2e-2)


def test_decode_attention_with_more_ctas_than_resident_slots(k, ref):
    """So many sequences that even one key range each is more CTAs than are resident
    at once: the policy then cuts every sequence into a few ranges (so that a last
    round with a few CTAs does not cost a whole one), and the result must not care."""
    nq, nkv, d, page = 16, 8, 128, 16
    seqs = 2 * k.sm_count // nkv + 3                          # a few CTAs past the resident slots
    seq_ctx = [1600 + 37 * (i % 7) for i in range(seqs)]
    assert k.decode_attention_splits(seqs, nq, nkv, max(seq_ctx)) > 1
    assert k.decode_attention_splits(seqs, nq, nkv, 600) == 1            # short sequences: a prologue more costs more
    assert k.decode_attention_splits(2 * k.sm_count // nkv, nq, nkv, 4096) == 1
    pages = sum((c + page - 1) // page for c in seq_ctx) + 1
    table, positions, seq_of_token, q_start, ctx_len = _paged_setup(seq_ctx, [1] * seqs, page, pages, seed=21)
    q = rnd(seqs, nq * d, dtype=torch.bfloat16, seed=22)
    kc = rnd(pages, nkv, page, d, dtype=torch.bfloat16, seed=23)
    vc = rnd(pages, nkv, page, d, dtype=torch.bfloat16, seed=24)
    out = torch.full((seqs, nq * d), float("nan"), dtype=torch.bfloat16, device="cuda")
    exp = torch.empty_like(out)
    args = (table, q_start, ctx_len, seq_of_token, positions, nq, nkv, d, page, 1.0 / math.sqrt(d), None, 1,
            max(seq_ctx), 1)
    k.attention(q, kc, vc, out, *args)
    ref.attention(q, kc, vc, exp, *args)
    k.check_error_word()
    close(out, exp, torch.bfloat16, "decode attention, more CTAs than slots", rel=1.2e-2)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("needle,window", [(0, None), (3, None), (255, None), (256, None), (700, None),
                                           (1000 - 40, 40), (1000 - 41, 40)])
def test_attention_finds_one_far_key(k, dtype, needle, window):
    """One key among a thousand matches the query; the output must be that key's
    value -- or, if the key lies just outside the window, must not be."""
    nq, nkv, d, page = 2, 1, 64, 16
    ctx = 1000
    pages = 80
    table, positions, seq_of_token, q_start, ctx_len = _paged_setup([ctx], [1], page, pages, seed=13)
    q = torch.zeros(1, nq * d, dtype=dtype, device="cuda")
    q[0, 5] = 40.0
    q[0, d + 5] = 40.0
    kc = (0.01 * rnd(pages, nkv, page, d, seed=14)).to(dtype)
    vc = rnd(pages, nkv, page, d, dtype=dtype, seed=15)
    pg = int(table[0, needle // page])
    kc[pg, 0, needle % page, 5] = 40.0
    out = torch.empty(1, nq * d, dtype=dtype, device="cuda")
    k.attention(q, kc, vc, out, table, q_start, ctx_len, seq_of_token, positions, nq, nkv, d, page,
                1.0 / math.sqrt(d), window, 1, ctx)
    target = vc[pg, 0, needle % page, :].float()
    visible = window is None or needle > (ctx - 1) - window
    got = out.float().view(nq, d)
    for h in range(nq):
        err = float((got[h] - target).abs().max())
        if visible:
            assert err < 2e-2, f"head {h}: the key at {needle} was not found (err {err})"
        else:
            assert err > 0.3, f"head {h}: the key at {needle} lies outside the window but was used"


@pytest.mark.parametrize("dtype", DTYPES)
def test_swiglu_and_gather(k, ref, dtype):
    gu = rnd(13, 2 * 176, dtype=dtype, seed=16, scale=3.0)
    out = torch.empty(13, 176, dtype=dtype, device="cuda")
    exp = torch.empty_like(out)
    k.swiglu(gu, out)
    ref.swiglu(gu, exp)
    close(out, exp, dtype, "swiglu", rel=3e-6 if dtype == torch.float32 else 8e-3)
    x = rnd(29, 80, seed=17)
    rows = torch.tensor([28, 0, 7, 7], dtype=torch.int32, device="cuda")
    g = torch.empty(4, 80, device="cuda")
    k.gather_rows(x, rows, g)
    assert torch.equal(g, x[rows.long()])


def test_cast_and_add(k):
    x = rnd(1001, dtype=torch.float32, seed=18)
    y = torch.empty(1001, dtype=torch.bfloat16, device="cuda")
    k.cast(x, y)
    assert torch.equal(y, x.to(torch.bfloat16))
    acc = rnd(1001, seed=19)
    exp = acc + y.float()
    k.add_into(acc, y)
    assert torch.equal(acc, exp)


@pytest.mark.parametrize("vocab", [301, 4096, 151936])
def test_sample_greedy_and_ties(k, vocab):
    logits = rnd(5, vocab, seed=20)
    logits[1, 17] = 50.0
    logits[1, 200] = 50.0          # tie: the lower id wins
    logits[2, vocab - 1] = 60.0
    logits[3] = 0.0                # all equal: id 0
    out = torch.empty(5, dtype=torch.int32, device="cuda")
    k.sample(logits, None, None, out)
    exp = [int(torch.nonzero(logits[r] == logits[r].max())[0, 0]) for r in range(5)]
    assert out.tolist() == exp
    assert exp[1] == 17 and exp[2] == vocab - 1 and exp[3] == 0


@pytest.mark.parametrize("vocab", [301, 151936])
def test_sample_temperature(k, vocab):
    R = 64
    logits = rnd(R, vocab, seed=21, scale=2.0)
    temps = torch.full((R,), 0.7, device="cuda")
    temps[0] = 0.0                                     # a greedy row beside sampled ones
    uni = torch.rand(R, generator=torch.Generator(device="cuda").manual_seed(22), device="cuda")
    uni[1], uni[2] = 0.0, 0.99999994
    out = torch.empty(R, dtype=torch.int32, device="cuda")
    k.sample(logits, temps, uni, out)
    got = out.tolist()
    assert got[0] == int(logits[0].argmax())
    for r in range(1, R):
        p = torch.exp((logits[r].double() - logits[r].double().max()) / 0.7)
        cdf = torch.cumsum(p, 0) / p.sum()
        u = float(uni[r])
        lo = float(cdf[got[r] - 1]) if got[r] > 0 else 0.0
        hi = float(cdf[got[r]])
        # the chosen id's interval of the CDF holds u, up to 32-bit rounding of the sums
        assert lo - 1e-4 <= u <= hi + 1e-4, f"row {r}: id {got[r]} covers [{lo}, {hi}], u = {u}"


@pytest.mark.parametrize("M", [1, 8, 16, 17, 33, 64, 65, 128, 300])
@pytest.mark.parametrize("N,K", [(203, 96), (256, 512), (1000, 1000), (384, 4096)])
def test_linear_tensor_cores(k, ref, M, N, K):
    """The tcgen05 kernel at sizes that are no multiple of its tiles: rows and
    features past the edge, a K tail, K ranges split over CTAs for few rows
    (through global scratch), and enough K blocks that the ring of stages wraps
    several times."""
    _linear_tensor_cores(k, ref, M, N, K)


def _linear_tensor_cores(k, ref, M, N, K):
    x = rnd(M, K, dtype=torch.bfloat16, seed=30)
    w = rnd(N, K, dtype=torch.bfloat16, seed=31, scale=0.05)
    before = k.tensor_core_calls
    for odtype in (torch.bfloat16, torch.float32):
        out = torch.full((M, N), float("nan"), dtype=odtype, device="cuda")
        exp = torch.empty_like(out)
        k.linear(x, w, out)
        ref.linear(x, w, exp)
        close(out, exp, odtype, f"tensor-core linear -> {odtype}", rel=2e-5 if odtype == torch.float32 else 8e-3)
    res = rnd(M, N, seed=32)
    exp_res = torch.empty_like(res)
    ref.linear(x, w, exp_res, residual=res)
    k.linear(x, w, res, residual=res)
    close(res, exp_res, torch.float32, "tensor-core linear + residual in place", rel=2e-5)
    assert k.tensor_core_calls == before + 3, "the tensor-core kernel refused an aligned shape"
    k.check_error_word()
    # a view with a row stride (the q part of a packed projection, a slice of the weights)
    wide = rnd(M, K + 64, dtype=torch.bfloat16, seed=33)
    out = torch.empty(M, 128, dtype=torch.float32, device="cuda")
    exp = torch.empty_like(out)
    k.linear(wide[:, 64:], w[:128], out)
    ref.linear(wide[:, 64:], w[:128], exp)
    close(out, exp, torch.float32, "tensor-core linear on views", rel=2e-5)


@pytest.mark.parametrize("M,N,K", [(1300, 4096, 1024), (2000, 5120, 5160), (300, 1000, 1000), (257, 512, 8192),
                                   (1280, 4096, 17408),                       # shared out whatever the pairs could do
                                   (2100, 768, 512), (4500, 1024, 264),       # more than one band of row blocks
                                   (512, 4096, 264), (1024, 6144, 136), (400, 384, 512)])   # tiles of 128 columns
@pytest.mark.parametrize("pairs", ["never", "policy"])
def test_linear_shares_out_a_thin_last_round(k, ref, M, N, K, pairs):
    """Many rows whose tiles leave a last round that fills a quarter of the SMs or
    less: the K blocks of those tiles are dealt out to all SMs and the partial
    sums added by the tile's first CTA.  Same result as whole tiles up to the
    order of 32-bit sums, launch after launch (the counters are left at zero).
    With pairs of CTAs allowed the plan gives some of these shapes to them
    instead; the one with 272 K blocks stays with single CTAs and its shared-out round."""
    k.pairs_of_ctas(pairs)
    try:
        if (M, N, K) == (1280, 4096, 17408):
            assert k.lib.chibi_gemm_many_rows_plan(M, N, K) == 256
        _linear_shares_out_a_thin_last_round(k, ref, M, N, K)
    finally:
        k.pairs_of_ctas("policy")


def _linear_shares_out_a_thin_last_round(k, ref, M, N, K):
    x = rnd(M, K, dtype=torch.bfloat16, seed=36)
    w = rnd(N, K, dtype=torch.bfloat16, seed=37, scale=0.05)
    exp = torch.empty(M, N, dtype=torch.float32, device="cuda")
    if K > 8192:
        # so long a sum in 32-bit is itself off by about the bound below: the exact sums instead
        exp.copy_(x.double() @ w.double().t())
    else:
        ref.linear(x, w, exp)
    # The bound of the sums up to 8,192 terms that the other cases have; the tensor core adds its
    # products to the 32-bit accumulator without rounding to nearest, so the error of a sum grows
    # with its length (measured against the exact sums at 17,408 terms: 2.1e-5 of the largest value).
    bound = 2e-5 * max(1.0, K / 8192)
    whole = torch.empty_like(exp)
    k.share_out_last_round(False)
    try:
        k.linear(x, w, whole)
    finally:
        k.share_out_last_round(True)
    close(whole, exp, torch.float32, "whole tiles", rel=bound)
    for launch in range(3):
        out = torch.full((M, N), float("nan"), dtype=torch.float32, device="cuda")
        k.linear(x, w, out)
        close(out, exp, torch.float32, f"last round shared out, launch {launch}", rel=bound)
    res = rnd(M, N, seed=38)
    exp_res = res + exp
    k.linear(x, w, res, residual=res)
    close(res, exp_res, torch.float32, "shared out + residual in place", rel=bound)
    out16 = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    exp16 = torch.empty_like(out16)
    k.linear(x, w, out16)
    ref.linear(x, w, exp16)
    close(out16, exp16, torch.bfloat16, "shared out -> bfloat16", rel=8e-3)
    k.check_error_word()


@pytest.mark.parametrize("M,hidden,K,wide", [(300, 512, 384, 768), (130, 256, 1024, 512), (2000, 1024, 520, 2560),
                                             (512, 4096, 136, 1024), (1024, 2048, 264, 6144)])   # tiles of 128 columns
@pytest.mark.parametrize("wdtype", DTYPES)
def test_linear_folds_the_norm_that_follows(k, ref, M, hidden, K, wide, wdtype):
    """Many rows: the product that completes the residual also writes the RMSNorm of
    the new residual up to each row's factor, and the products that read it (plain
    and with SwiGLU) apply the factor to their sums; any other reader has it
    applied in place."""
    from chibillm_b200.kernels.ops import ScaledRows
    x = rnd(M, K, dtype=torch.bfloat16, seed=50)
    w = rnd(hidden, K, dtype=torch.bfloat16, seed=51, scale=0.05)
    res = rnd(M, hidden, seed=52, scale=3.0)
    nw = (1 + 0.1 * rnd(hidden, seed=53)).to(wdtype)
    eps, offset = 1e-5, 0.25
    exp_res = torch.empty_like(res)
    ref.linear(x, w, exp_res, residual=res)
    exp_normed = torch.empty(M, hidden, dtype=torch.float32, device="cuda")
    ref.rmsnorm(exp_res, nw, eps, offset, exp_normed)

    normed = torch.full((M, hidden), float("nan"), dtype=torch.bfloat16, device="cuda")
    scaled = k.linear_residual_norm(x, w, res, nw, eps, offset, normed)
    assert isinstance(scaled, ScaledRows), "the kernel refused shapes it is made for"
    close(res, exp_res, torch.float32, "residual", rel=2e-5)
    # the product that reads it
    w2 = rnd(wide, hidden, dtype=torch.bfloat16, seed=54, scale=0.05)
    out = torch.full((M, wide), float("nan"), dtype=torch.bfloat16, device="cuda")
    before = k.launches
    k.linear(scaled, w2, out)
    assert k.launches == before + 1, "the factor was not applied by the product itself"
    exp = torch.empty(M, wide, dtype=torch.float32, device="cuda")
    ref.linear(exp_normed, w2, exp)
    close(out, exp, torch.bfloat16, "product of rows with a factor", rel=1.2e-2)
    # ... with SwiGLU
    gate = rnd(wide // 2, hidden, dtype=torch.bfloat16, seed=55, scale=0.05)
    up = rnd(wide // 2, hidden, dtype=torch.bfloat16, seed=56, scale=0.05)
    act = torch.full((M, wide // 2), float("nan"), dtype=torch.bfloat16, device="cuda")
    assert k.linear_swiglu(scaled, k.interleave_gate_up(gate, up), act)
    gu = torch.empty(M, wide, dtype=torch.float32, device="cuda")
    ref.linear(exp_normed, torch.cat([gate, up]), gu)
    exp_act = torch.empty(M, wide // 2, dtype=torch.float32, device="cuda")
    ref.swiglu(gu, exp_act)
    close(act, exp_act, torch.bfloat16, "SwiGLU of rows with a factor", rel=1.2e-2)
    # a reader that is no product (here: a product the kernel for many rows does not take)
    narrow = rnd(40, hidden, dtype=torch.bfloat16, seed=57, scale=0.05)
    out2 = torch.empty(M, 40, dtype=torch.float32, device="cuda")
    k.linear(scaled, narrow, out2)
    exp2 = torch.empty_like(out2)
    ref.linear(exp_normed, narrow, exp2)
    close(out2, exp2, torch.float32, "factor applied in place first", rel=1.2e-2)
    close(normed, exp_normed, torch.bfloat16, "the norm's output after the factor", rel=8e-3)
    k.check_error_word()


@pytest.mark.parametrize("M,hidden,K,wide", [(256, 256, 64, 512), (300, 512, 1000, 768), (513, 1024, 520, 2560),
                                             (1000, 768, 4096, 512), (2048 + 17, 512, 264, 1024)])
def test_products_by_pairs_of_ctas(k, ref, M, hidden, K, wide):
    """Tiles of 256 x 256 and 256 x 128 by two CTAs (one tcgen05.mma of 256 rows for both) against the same
    products by single CTAs: the sums are added in the same order, so every output is the same
    bit for bit -- plain, onto the residual with the next norm's output, of rows with a factor,
    with SwiGLU; rows that end inside a tile's first or second half, one tile and many."""
    x = rnd(M, K, dtype=torch.bfloat16, seed=60)
    w = rnd(hidden, K, dtype=torch.bfloat16, seed=61, scale=0.05)
    res0 = rnd(M, hidden, seed=62, scale=3.0)
    nw = (1 + 0.1 * rnd(hidden, seed=63)).to(torch.bfloat16)
    w2 = rnd(wide, hidden, dtype=torch.bfloat16, seed=64, scale=0.05)
    gu = k.interleave_gate_up(rnd(wide // 2, hidden, dtype=torch.bfloat16, seed=65, scale=0.05),
                              rnd(wide // 2, hidden, dtype=torch.bfloat16, seed=66, scale=0.05))
    results = {}
    try:
        for mode in ("never", "always", "always narrow"):
            k.pairs_of_ctas(mode)
            plain = torch.full((M, hidden), float("nan"), dtype=torch.bfloat16, device="cuda")
            k.linear(x, w, plain)
            res = res0.clone()
            normed = torch.full((M, hidden), float("nan"), dtype=torch.bfloat16, device="cuda")
            scaled = k.linear_residual_norm(x, w, res, nw, 1e-5, 0.0, normed)
            assert scaled is not None, "the kernel refused shapes it is made for"
            out = torch.full((M, wide), float("nan"), dtype=torch.bfloat16, device="cuda")
            k.linear(scaled, w2, out)
            act = torch.full((M, wide // 2), float("nan"), dtype=torch.bfloat16, device="cuda")
            assert k.linear_swiglu(scaled, gu, act)
            k.check_error_word()
            ssq = scaled.ssq[:M * scaled.parts].view(M, scaled.parts).sum(1)
            results[mode] = (plain, res, normed.clone(), ssq, out, act)
    finally:
        k.pairs_of_ctas("policy")
    names = ("plain", "residual", "norm output", "sums of squares", "of rows with a factor", "SwiGLU")
    for mode in ("always", "always narrow"):
        for i, (what, a, b) in enumerate(zip(names, results["never"], results[mode])):
            assert torch.isfinite(a.float()).all(), what
            if i < 3:
                assert torch.equal(a, b), f"{what}: pairs of CTAs ({mode}) differ from single CTAs"
            else:
                # tiles of 128 or of 256 columns: the parts of a row's sum of squares are then added
                # in another order, and a factor may differ in its last bit
                close(a, b, torch.float32 if i == 3 else torch.bfloat16, what, rel=1e-5 if i == 3 else 8e-3)
                if i > 3:
                    assert (a == b).float().mean() > 0.995, f"{what}: pairs of CTAs ({mode}) differ from single CTAs"
    exp = torch.empty(M, hidden, dtype=torch.float32, device="cuda")
    ref.linear(x, w, exp)
    close(results["always"][0], exp, torch.bfloat16, "plain product by pairs", rel=8e-3)


def test_linear_falls_back_when_unaligned(k, ref):
    x = rnd(5, 100, dtype=torch.bfloat16, seed=34)      # K = 100 is no multiple of 8
    w = rnd(40, 100, dtype=torch.bfloat16, seed=35)
    out = torch.empty(5, 40, dtype=torch.float32, device="cuda")
    exp = torch.empty_like(out)
    before = k.tensor_core_calls
    k.linear(x, w, out)
    ref.linear(x, w, exp)
    assert k.tensor_core_calls == before
    close(out, exp, torch.float32, "fallback linear", rel=2e-5)


@pytest.mark.parametrize("M", [1, 8, 33, 64, 100, 128])
def test_split_product_with_fused_consumers(k, ref, M):
    """A product whose K range is split over CTAs, finished by the kernels that
    add the partial sums together with what follows: residual + RMSNorm, SwiGLU,
    per-head norm + rotation + cache append."""
    K = 4096
    k.fuse_split_products = True
    x = rnd(M, K, dtype=torch.bfloat16, seed=40)
    # residual + norm (and residual alone)
    N = 1024
    w = rnd(N, K, dtype=torch.bfloat16, seed=41, scale=0.05)
    nw = (1 + 0.1 * rnd(N, seed=42)).to(torch.bfloat16)
    res = rnd(M, N, seed=43)
    pending = k.linear_partial(x, w)
    assert pending is not None and pending.splits > 1
    got_res = res.clone()
    got_norm = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    k.reduce_residual_rmsnorm(pending, got_res, nw, 1e-5, 0.0, got_norm)
    exp_res = torch.empty_like(res)
    ref.linear(x, w, exp_res, residual=res)
    exp_norm = torch.empty_like(got_norm)
    ref.rmsnorm(exp_res, nw, 1e-5, 0.0, exp_norm)
    close(got_res, exp_res, torch.float32, "split product + residual", rel=2e-5)
    close(got_norm, exp_norm, torch.bfloat16, "split product + residual + norm", rel=8e-3)
    pending = k.linear(x, w, res, residual=res, defer=True)
    assert pending is not None
    pending.add_into(res)
    close(res, exp_res, torch.float32, "deferred residual add", rel=2e-5)
    # SwiGLU
    inter = 768
    wgu = rnd(2 * inter, K, dtype=torch.bfloat16, seed=44, scale=0.03)
    pending = k.linear_partial(x, wgu)
    assert pending is not None
    act = torch.full((M, inter), float("nan"), dtype=torch.bfloat16, device="cuda")
    k.reduce_swiglu(pending, act)
    gu = torch.empty(M, 2 * inter, dtype=torch.float32, device="cuda")
    ref.linear(x, wgu, gu)
    exp_act = torch.empty_like(act)
    ref.swiglu(gu, exp_act)
    close(act, exp_act, torch.bfloat16, "split product + SwiGLU", rel=8e-3)
    # per-head norm + rotation + append
    nq, nkv, d, page, pages = 6, 2, 64, 16, 40
    seq_ctx = [min(5 + 7 * i, 600) for i in range(M)]
    table, positions, seq_of_token, _, _ = _paged_setup(seq_ctx, [1] * M, page, max(pages, sum((c + 15) // 16 for c in seq_ctx) + 1), seed=45)
    pages = max(pages, int(table.max()) + 1)
    wqkv = rnd((nq + 2 * nkv) * d, K, dtype=torch.bfloat16, seed=46, scale=0.03)
    qn = (1 + 0.1 * rnd(d, seed=47)).to(torch.bfloat16)
    kn = (1 + 0.1 * rnd(d, seed=48)).to(torch.bfloat16)
    inv_freq = torch.pow(torch.tensor(1e6), -2 * torch.arange(d // 2, dtype=torch.float32) / d).cuda()
    pending = k.linear_partial(x, wqkv)
    assert pending is not None
    q_got = torch.full((M, nq * d), float("nan"), dtype=torch.bfloat16, device="cuda")
    kc = torch.zeros(pages, nkv, page, d, dtype=torch.bfloat16, device="cuda")
    vc = torch.zeros_like(kc)
    k.qk_norm_rope_append_partial(pending, q_got, kc, vc, qn, kn, inv_freq, d, 1e-6, 0.0, positions,
                                  seq_of_token, table, nq, nkv, d, page)
    qkv = torch.empty(M, (nq + 2 * nkv) * d, dtype=torch.float32, device="cuda")
    ref.linear(x, wqkv, qkv)
    q_exp = torch.empty(M, nq * d, dtype=torch.float32, device="cuda")
    kc_exp = torch.zeros(pages, nkv, page, d, dtype=torch.float32, device="cuda")
    vc_exp = torch.zeros_like(kc_exp)
    ref.qk_norm_rope_append(qkv, q_exp, kc_exp, vc_exp, qn, kn, inv_freq, d, 1e-6, 0.0, positions,
                            seq_of_token, table, nq, nkv, d, page)
    close(q_got, q_exp, torch.bfloat16, "split product -> q", rel=8e-3)
    close(kc, kc_exp, torch.bfloat16, "split product -> key cache", rel=8e-3)
    close(vc, vc_exp, torch.bfloat16, "split product -> value cache", rel=8e-3)
    k.check_error_word()


@pytest.mark.parametrize("M", [1, 8, 17, 64, 65, 300])
@pytest.mark.parametrize("inter,K", [(64, 512), (192, 4096), (768, 1000)])
def test_linear_swiglu(k, ref, M, inter, K):
    """SwiGLU inside the matrix product: the weights come as blocks of 64 gate
    rows and their 64 up rows; for few rows the CTAs of a cluster add their
    partial sums through distributed shared memory."""
    gate = rnd(inter, K, dtype=torch.bfloat16, seed=50, scale=0.05)
    up = rnd(inter, K, dtype=torch.bfloat16, seed=51, scale=0.05)
    x = rnd(M, K, dtype=torch.bfloat16, seed=52)
    w = k.interleave_gate_up(gate, up)
    assert w is not None and w.shape == (2 * inter, K)
    assert torch.equal(w[:64], gate[:64]) and torch.equal(w[64:128], up[:64])
    out = torch.full((M, inter), float("nan"), dtype=torch.bfloat16, device="cuda")
    assert k.linear_swiglu(x, w, out)
    gu = torch.empty(M, 2 * inter, dtype=torch.float32, device="cuda")
    ref.linear(x, torch.cat([gate, up]), gu)
    exp = torch.empty_like(out)
    ref.swiglu(gu, exp)
    close(out, exp, torch.bfloat16, "product + SwiGLU", rel=8e-3)
    k.check_error_word()
    assert k.interleave_gate_up(gate[:40], up[:40]) is None


@pytest.mark.parametrize("nq,nkv,d,window", [(8, 2, 128, None), (4, 1, 64, None), (8, 2, 128, 1500)])
@pytest.mark.parametrize("seq_ctx,q_lens", [([3000], [130]), ([2600, 1100], [40, 3])])
def test_prompt_attention_with_key_ranges(k, ref, nq, nkv, d, window, seq_ctx, q_lens):
    """Few query rows over a long context: the tcgen05 kernel cuts the keys of a row
    tile into ranges, one CTA each, and a second kernel puts the ranges together
    (ranges may be empty for the tile with fewer keys); same result as the plain one."""
    page = 16
    assert k.prompt_attention_key_ranges(len(seq_ctx), nq, nkv, max(q_lens), max(seq_ctx)) > 1
    assert k.prompt_attention_key_ranges(len(seq_ctx), nq, nkv, max(q_lens), 700) == 1
    assert k.prompt_attention_key_ranges(40, nq, nkv, 512, 8192) == 1
    pages = sum((c + page - 1) // page for c in seq_ctx) + 3
    table, positions, seq_of_token, q_start, ctx_len = _paged_setup(seq_ctx, q_lens, page, pages, seed=70)
    T = sum(q_lens)
    q = rnd(T, nq * d, dtype=torch.bfloat16, seed=71)
    kc = torch.full((pages, nkv, page, d), float("nan"), dtype=torch.bfloat16, device="cuda")
    vc = torch.full((pages, nkv, page, d), float("nan"), dtype=torch.bfloat16, device="cuda")
    for s, c in enumerate(seq_ctx):
        idx = torch.arange(c, device="cuda")
        pg = table[s, idx // page].long()
        kc[pg, :, idx % page, :] = rnd(c, nkv, d, dtype=torch.bfloat16, seed=2100 + s)
        vc[pg, :, idx % page, :] = rnd(c, nkv, d, dtype=torch.bfloat16, seed=6100 + s)
    args = (table, q_start, ctx_len, seq_of_token, positions, nq, nkv, d, page, 1.0 / math.sqrt(d), window,
            max(q_lens), max(seq_ctx), min(q_lens))
    exp = torch.empty(T, nq * d, dtype=torch.bfloat16, device="cuda")
    ref.attention(q, kc, vc, exp, *args)
    out = torch.full((T, nq * d), float("nan"), dtype=torch.bfloat16, device="cuda")
    k.attention(q, kc, vc, out, *args)
    k.check_error_word()
    close(out, exp, torch.bfloat16, "prompt attention with key ranges", rel=1.2e-2)


@pytest.mark.parametrize("nq,nkv,d,window", [(8, 2, 128, None), (5, 1, 128, 200), (4, 4, 64, None), (6, 2, 64, 130)])
@pytest.mark.parametrize("page", [8, 16, 64])
def test_attention_tcgen05_prompts(k, ref, nq, nkv, d, window, page):
    """Prompt attention on tcgen05 (S and the per-tile output in TMEM, V as the
    MN-major operand): several 128-key tiles, a portion that continues a long
    context, rows of several tokens and heads in one tile, a window; and the same
    through the mma.sync kernel."""
    seq_ctx, q_lens = [700, 300, 130], [700, 45, 2]
    pages = sum((c + page - 1) // page for c in seq_ctx) + 3
    table, positions, seq_of_token, q_start, ctx_len = _paged_setup(seq_ctx, q_lens, page, pages, seed=60)
    T = sum(q_lens)
    q = rnd(T, nq * d, dtype=torch.bfloat16, seed=61)
    kc = torch.full((pages, nkv, page, d), float("nan"), dtype=torch.bfloat16, device="cuda")
    vc = torch.full((pages, nkv, page, d), float("nan"), dtype=torch.bfloat16, device="cuda")
    for s, c in enumerate(seq_ctx):
        idx = torch.arange(c, device="cuda")
        pg = table[s, idx // page].long()
        kc[pg, :, idx % page, :] = rnd(c, nkv, d, dtype=torch.bfloat16, seed=2000 + s)
        vc[pg, :, idx % page, :] = rnd(c, nkv, d, dtype=torch.bfloat16, seed=6000 + s)
    args = (table, q_start, ctx_len, seq_of_token, positions, nq, nkv, d, page, 1.0 / math.sqrt(d), window,
            max(q_lens), max(seq_ctx), min(q_lens))
    exp = torch.empty(T, nq * d, dtype=torch.bfloat16, device="cuda")
    ref.attention(q, kc, vc, exp, *args)
    outs = {}
    for tc, variant in ((True, 1), (True, 2), (False, 0)):      # one and two query tiles per CTA; mma.sync
        k.use_tcgen05_attention = tc
        k.tcgen05_attention_variant = variant
        out = torch.full((T, nq * d), float("nan"), dtype=torch.bfloat16, device="cuda")
        before = k.launches
        k.attention(q, kc, vc, out, *args)
        k.check_error_word()
        close(out, exp, torch.bfloat16, f"prompt attention (tcgen05={tc}, variant {variant})", rel=1.2e-2)
        outs[(tc, variant)] = out
    k.use_tcgen05_attention = True
    k.tcgen05_attention_variant = 0


@pytest.mark.parametrize("nq,nkv,window,append", [(32, 8, None, True), (8, 2, 100, True), (6, 1, None, True),
                                                  (8, 2, None, False)])
def test_decode_attention_from_partial_sums(k, ref, nq, nkv, window, append):
    """Decode attention that finishes the q | k | v product itself (sum of the
    partial sums, per-head norm, rotation, append of the new key and value) against
    the plain restatement of product, norm, rotation, append and attention, and
    against the two kernels it replaces, on sequences that end at and next to page
    edges."""
    d, page, K = 128, 16, 1024
    seq_ctx = [1, 16, 17, 129, 300, 640, 33, 48]
    S = len(seq_ctx)
    pages = sum((c + page - 1) // page for c in seq_ctx) + 2
    table, positions, seq_of_token, q_start, ctx_len = _paged_setup(seq_ctx, [1] * S, page, pages, seed=80)
    x = rnd(S, K, dtype=torch.bfloat16, seed=81)
    width = (nq + 2 * nkv) * d if append else nq * d
    w = rnd(width, K, dtype=torch.bfloat16, seed=82, scale=0.05)
    qn = (1 + 0.1 * rnd(d, seed=83)).to(torch.bfloat16)
    kn = (1 + 0.1 * rnd(d, seed=84)).to(torch.bfloat16)
    inv_freq = torch.pow(torch.tensor(1e6), -2 * torch.arange(d // 2, dtype=torch.float32) / d).cuda()
    kc0 = rnd(pages, nkv, page, d, dtype=torch.bfloat16, seed=85)
    vc0 = rnd(pages, nkv, page, d, dtype=torch.bfloat16, seed=86)
    scale = 1.0 / math.sqrt(d)

    kc, vc = kc0.clone(), vc0.clone()
    pending = k.linear_partial(x, w)
    assert pending is not None and pending.splits > 1
    q = torch.empty(S, nq * d, dtype=torch.bfloat16, device="cuda")
    k.qk_norm_rope_append_partial(pending, q, kc if append else None, vc if append else None, qn, kn, inv_freq, d,
                                  1e-6, 0.0, positions, seq_of_token, table if append else None, nq, nkv, d, page)
    exp = torch.empty(S, nq * d, dtype=torch.bfloat16, device="cuda")
    k.attention(q, kc, vc, exp, table, q_start, ctx_len, seq_of_token, positions, nq, nkv, d, page, scale, window,
                1, max(seq_ctx), 1)

    kc2, vc2 = kc0.clone(), vc0.clone()
    pending = k.linear_partial(x, w)
    got = torch.full((S, nq * d), float("nan"), dtype=torch.bfloat16, device="cuda")
    assert k.attention_decode_from_partial(pending, kc2, vc2, got, table, q_start, ctx_len, nq, nkv, d, page, scale,
                                           window, max(seq_ctx), qn, kn, inv_freq, d, 1e-6, 0.0, append)
    k.check_error_word()
    close(got, exp, torch.bfloat16, "decode attention from the partial sums", rel=8e-3)
    close(kc2, kc, torch.bfloat16, "key cache", rel=8e-3)
    assert torch.equal(vc2, vc), "value cache"

    # the plain restatement, in 32-bit from the same bfloat16 inputs
    kc3, vc3 = kc0.clone(), vc0.clone()
    qkv = torch.empty(S, width, dtype=torch.float32, device="cuda")
    ref.linear(x, w, qkv)
    q3 = torch.empty(S, nq * d, dtype=torch.float32, device="cuda")
    ref.qk_norm_rope_append(qkv, q3, kc3 if append else None, vc3 if append else None, qn, kn, inv_freq, d, 1e-6,
                            0.0, positions, seq_of_token, table if append else None, nq, nkv, d, page)
    plain = torch.empty(S, nq * d, dtype=torch.float32, device="cuda")
    ref.attention(q3, kc3, vc3, plain, table, q_start, ctx_len, seq_of_token, positions, nq, nkv, d, page, scale,
                  window, 1, max(seq_ctx))
    close(got, plain, torch.bfloat16, "decode attention from the partial sums vs the plain restatement", rel=1.2e-2)
    close(kc2, kc3, torch.bfloat16, "key cache vs the plain restatement", rel=8e-3)
    close(vc2, vc3, torch.bfloat16, "value cache vs the plain restatement", rel=8e-3)


@pytest.mark.parametrize("nq,nkv,norms,wdtype,append", [(6, 2, True, torch.bfloat16, True),
                                                        (24, 4, True, torch.bfloat16, True),     # tiles of one head
                                                        (5, 1, True, torch.float32, True),       # an odd number of heads
                                                        (4, 1, True, torch.float32, True),
                                                        (8, 4, False, torch.bfloat16, True),
                                                        (4, 2, True, torch.bfloat16, False)])
@pytest.mark.parametrize("seq_ctx,q_lens,scaled", [([70, 8, 300], [40, 1, 133], False),
                                                   ([257, 130, 64, 90], [257, 2, 64, 77], True)])
@pytest.mark.parametrize("pairs", ["policy", "always", "always narrow"])
def test_product_that_finishes_its_heads(k, ref, nq, nkv, norms, wdtype, append, seq_ctx, q_lens, scaled, pairs):
    """The q | k | v product of many rows whose epilogue normalises and rotates the
    heads and writes q and the cache entries (head size 128), against the plain
    product followed by the plain norm + rotation + append; with and without a row
    factor left by the norm before (``ScaledRows``); rows that end inside a tile; by single
    CTAs and (400 rows, widths of whole tiles of 256) by pairs of CTAs."""
    k.pairs_of_ctas(pairs)
    try:
        _product_that_finishes_its_heads(k, ref, nq, nkv, norms, wdtype, append, seq_ctx, q_lens, scaled)
    finally:
        k.pairs_of_ctas("policy")


def _product_that_finishes_its_heads(k, ref, nq, nkv, norms, wdtype, append, seq_ctx, q_lens, scaled):
    from chibillm_b200.kernels.ops import ScaledRows
    d, page, K = 128, 16, 520
    T = sum(q_lens)
    pages = sum((c + page - 1) // page for c in seq_ctx) + 3
    table, positions, seq_of_token, _, _ = _paged_setup(seq_ctx, q_lens, page, pages, seed=120)
    width = (nq + 2 * nkv) * d if append else nq * d
    x = rnd(T, K, dtype=torch.bfloat16, seed=121)
    w = rnd(width, K, dtype=torch.bfloat16, seed=122, scale=0.05)
    qn = (1 + 0.1 * rnd(d, seed=123)).to(wdtype) if norms else None
    kn = (1 + 0.1 * rnd(d, seed=124)).to(wdtype) if norms else None
    inv_freq = torch.pow(torch.tensor(1e6), -2 * torch.arange(d // 2, dtype=torch.float32) / d).cuda()
    kc0 = rnd(pages, nkv, page, d, dtype=torch.bfloat16, seed=125)
    vc0 = rnd(pages, nkv, page, d, dtype=torch.bfloat16, seed=126)

    given, x_plain = x, x.float()
    if scaled:
        parts, n, eps = 3, 4 * K, 1e-5
        ssq = (rnd(T, parts, seed=127).abs() * n).contiguous()
        given = ScaledRows(k, x, ssq, parts, eps, n)
        x_plain = x.float() * torch.rsqrt(ssq.sum(dim=1, keepdim=True) / n + eps)

    cos_sin = torch.full((T, d), float("nan"), dtype=torch.float32, device="cuda")
    k.rope_table(positions, inv_freq, d, cos_sin)
    angles = positions.float()[:, None] * inv_freq[None, :]
    assert torch.equal(cos_sin[:, :d // 2], torch.cos(angles)) or float((cos_sin[:, :d // 2] - torch.cos(angles)).abs().max()) < 1e-6
    assert float((cos_sin[:, d // 2:] - torch.sin(angles)).abs().max()) < 1e-6
    slots = None
    if append:
        slots = torch.full((T,), -7, dtype=torch.int64, device="cuda")
        k.cache_slots(positions, seq_of_token, None, table, nkv, page, pages, d, slots)
        exp_slots = (table[seq_of_token.long(), (positions // page).long()].long() * nkv * page + positions.long() % page) * d
        assert torch.equal(slots, exp_slots)

    q = torch.full((T, nq * d), float("nan"), dtype=torch.bfloat16, device="cuda")
    kc, vc = kc0.clone(), vc0.clone()
    assert k.linear_heads(given, w, q, kc if append else None, vc if append else None, qn, kn, cos_sin, slots,
                          nq, nkv, d, page, 1e-6, 0.0)
    k.check_error_word()

    qkv = x_plain @ w.float().t()
    q_exp = torch.empty(T, nq * d, dtype=torch.float32, device="cuda")
    kc_exp, vc_exp = kc0.float(), vc0.float()
    ref.qk_norm_rope_append(qkv, q_exp, kc_exp if append else None, vc_exp if append else None, qn, kn, inv_freq,
                            d, 1e-6, 0.0, positions, seq_of_token, table if append else None, nq, nkv, d, page)
    close(q, q_exp, torch.bfloat16, "heads from the product: q", rel=8e-3)
    if append:
        close(kc, kc_exp, torch.bfloat16, "heads from the product: key cache", rel=8e-3)
        close(vc, vc_exp, torch.bfloat16, "heads from the product: value cache", rel=8e-3)
        # slots of tokens that were not in the step are untouched
        written = torch.zeros(pages * nkv * page, dtype=torch.bool, device="cuda")
        for h in range(nkv):
            written[(slots // d + h * page).long()] = True
        untouched = ~written.view(pages, nkv, page)
        assert torch.equal(kc[untouched], kc0[untouched]) and torch.equal(vc[untouched], vc0[untouched])


def test_product_that_finishes_its_heads_refuses_what_it_does_not_take(k):
    """Few rows, another head size, a width that does not match the heads: False, nothing runs."""
    d, K = 128, 256
    cos_sin = torch.zeros(300, d, device="cuda")
    x = rnd(300, K, dtype=torch.bfloat16, seed=1)
    q = torch.zeros(300, 3 * d, dtype=torch.bfloat16, device="cuda")
    w = rnd(4 * d, K, dtype=torch.bfloat16, seed=2)
    assert not k.linear_heads(x, w, q, None, None, None, None, cos_sin, None, 3, 0, d, 16, 1e-6, 0.0)
    assert not k.linear_heads(x[:64], w[:3 * d], q[:64], None, None, None, None, cos_sin[:64], None, 3, 0, d, 16,
                              1e-6, 0.0)
    assert not k.finishes_heads(64, 128, 128, torch.bfloat16)
    assert not k.finishes_heads(300, 64, 64, torch.bfloat16)
    assert not k.finishes_heads(300, 128, 64, torch.bfloat16)
    assert not k.finishes_heads(300, 128, 128, torch.float32)
    assert float(q.abs().max()) == 0.0


def test_a_token_without_a_page_is_skipped_and_reported(k):
    """A block table without a page for some positions: the slot table says -1 for
    those tokens, the product writes their q and nothing else, every other token's
    cache entries are written, and the error word names the append."""
    from chibillm_b200.kernels.ops import KernelError
    nq, nkv, d, page, K = 4, 2, 128, 16, 256
    seq_ctx, q_lens = [100, 90], [100, 90]
    T = sum(q_lens)
    pages = 16
    table, positions, seq_of_token, _, _ = _paged_setup(seq_ctx, q_lens, page, pages, seed=130)
    table[1, 2] = -1                                  # positions 32..47 of the second sequence
    table[1, 4] = pages + 5                           # positions 64..79: a page that is not there
    bad = (seq_of_token == 1) & (((positions >= 32) & (positions < 48)) | ((positions >= 64) & (positions < 80)))
    slots = torch.full((T,), 123, dtype=torch.int64, device="cuda")
    k.cache_slots(positions, seq_of_token, None, table, nkv, page, pages, d, slots)
    assert torch.equal(slots < 0, bad) and int(bad.sum()) == 32
    inv_freq = torch.pow(torch.tensor(1e4), -2 * torch.arange(d // 2, dtype=torch.float32) / d).cuda()
    cos_sin = torch.empty(T, d, dtype=torch.float32, device="cuda")
    k.rope_table(positions, inv_freq, d, cos_sin)
    x = rnd(T, K, dtype=torch.bfloat16, seed=131)
    w = rnd((nq + 2 * nkv) * d, K, dtype=torch.bfloat16, seed=132, scale=0.05)
    q = torch.full((T, nq * d), float("nan"), dtype=torch.bfloat16, device="cuda")
    kc = torch.full((pages, nkv, page, d), 7.0, dtype=torch.bfloat16, device="cuda")
    vc = torch.full_like(kc, 7.0)
    assert k.linear_heads(x, w, q, kc, vc, None, None, cos_sin, slots, nq, nkv, d, page, 1e-6, 0.0)
    with pytest.raises(KernelError) as e:
        k.check_error_word()
    assert "append" in str(e.value)
    assert not bool(torch.isnan(q.float()).any())
    written = (kc != 7.0).any(dim=-1)                 # [pages, nkv, page]: slots that hold a new key
    assert int(written.sum()) == (T - 32) * nkv
    assert int((vc != 7.0).any(dim=-1).sum()) == (T - 32) * nkv
    k.check_error_word()                              # the word was cleared: nothing new


def test_a_pending_sum_that_was_overwritten_is_refused(k):
    """Split products take two scratch arrays in turn: the third one started
    writes over the first one's sums, and reading those then must raise."""
    from chibillm_b200.kernels.ops import KernelError
    k.fuse_split_products = True
    x = rnd(4, 4096, dtype=torch.bfloat16, seed=90)
    w = rnd(1024, 4096, dtype=torch.bfloat16, seed=91, scale=0.05)
    res = rnd(4, 1024, seed=92)
    first = k.linear_partial(x, w)
    second = k.linear_partial(x, w)
    assert first is not None and second is not None and first.splits > 1
    good = res.clone()
    first.add_into(good)                    # two products outstanding: both are still good
    third = k.linear_partial(x, w)
    with pytest.raises(KernelError) as e:
        first.add_into(res.clone())
    assert "overwritten" in str(e.value)
    a, b = res.clone(), res.clone()
    second.add_into(a)
    third.add_into(b)
    assert torch.equal(a, good) and torch.equal(b, good)
    k.check_error_word()
