"""The plain C++ restatements of the device operations, two ways round.

Without a GPU: each C++ loop against the PyTorch restatement of the same
operation (tests/reference_ops.py), so that two independent plain readings of
the reference's formulas have to agree.  With a GPU: each CUDA kernel against
the C++ loop, at small sizes that are no multiple of anything.
"""
import math

import pytest
import torch

from cpp_reference import CppReferenceKernels
from reference_ops import ReferenceKernels


@pytest.fixture(scope="module")
def cpp():
    return CppReferenceKernels()


@pytest.fixture(scope="module")
def plain():
    return ReferenceKernels()


def rnd(*shape, seed=0, scale=1.0, device="cpu", dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype).to(device)


def close(a, b, tol, what):
    a, b = a.float().cpu(), b.float().cpu()
    scale = float(b.abs().max()) + 1e-30
    worst = float((a - b).abs().max())
    assert torch.isfinite(a).all(), f"{what}: not finite"
    assert worst <= tol * scale, f"{what}: max |diff| {worst:.3e} > {tol:.1e} * {scale:.3e}"


def paged(seq_ctx, q_lens, page_size, num_pages, seed, device):
    """Block tables through shuffled pages; the last q_lens tokens of each sequence are the step's."""
    perm = torch.randperm(num_pages, generator=torch.Generator().manual_seed(seed)).tolist()
    width = max((c + page_size - 1) // page_size for c in seq_ctx)
    table = torch.full((len(seq_ctx), width), -1, dtype=torch.int32)
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
    dev = lambda v: torch.tensor(v, dtype=torch.int32, device=device)
    return table.to(device), dev(positions), dev(seq_of_token), dev(q_start), dev(seq_ctx)


def fill_caches(table, seq_ctx, pages, nkv, page, d, device, dtype=torch.float32, other=float("nan")):
    """Random keys and values at every held position; `other` in every slot that no sequence holds."""
    kc = torch.full((pages, nkv, page, d), other, dtype=dtype, device=device)
    vc = torch.full((pages, nkv, page, d), other, dtype=dtype, device=device)
    for s, c in enumerate(seq_ctx):
        idx = torch.arange(c, device=device)
        pg = table[s, idx // page].long()
        kc[pg, :, idx % page, :] = rnd(c, nkv, d, seed=1000 + s, device=device, dtype=dtype)
        vc[pg, :, idx % page, :] = rnd(c, nkv, d, seed=5000 + s, device=device, dtype=dtype)
    return kc, vc


# ---------------------------------------------------------------- without a GPU: C++ against PyTorch

def test_cpp_embed_norm_linear_swiglu_gather(cpp, plain):
    table = rnd(53, 24, seed=1)
    tokens = torch.tensor([0, 52, 7, 7, 31], dtype=torch.int32)
    a, b = torch.empty(5, 24), torch.empty(5, 24)
    cpp.embed(tokens, table, a)
    plain.embed(tokens, table, b)
    assert torch.equal(a, b)

    x, w = rnd(11, 40, seed=2, scale=3.0), 1 + 0.1 * rnd(40, seed=3)
    a, b = torch.empty(11, 40), torch.empty(11, 40)
    for eps, offset in ((1e-6, 0.0), (1e-3, 1.0)):
        cpp.rmsnorm(x, w, eps, offset, a)
        plain.rmsnorm(x, w, eps, offset, b)
        close(a, b, 2e-6, "rmsnorm")

    x, w, res = rnd(7, 40, seed=4), rnd(19, 40, seed=5, scale=0.2), rnd(7, 19, seed=6)
    a, b = torch.empty(7, 19), torch.empty(7, 19)
    for residual in (None, res):
        cpp.linear(x, w, a, residual=residual)
        plain.linear(x, w, b, residual=residual)
        close(a, b, 2e-6, "linear")

    gu = rnd(9, 2 * 22, seed=7, scale=3.0)
    a, b = torch.empty(9, 22), torch.empty(9, 22)
    cpp.swiglu(gu, a)
    plain.swiglu(gu, b)
    close(a, b, 2e-6, "swiglu")

    rows = torch.tensor([8, 0, 3, 3], dtype=torch.int32)
    a, b = torch.empty(4, 44), torch.empty(4, 44)
    cpp.gather_rows(gu, rows, a)
    plain.gather_rows(gu, rows, b)
    assert torch.equal(a, b)


@pytest.mark.parametrize("nq,nkv,d,rot,norms", [(6, 2, 48, 48, True), (4, 4, 16, 8, True), (5, 1, 32, 32, False),
                                                (2, 1, 32, 0, True)])
def test_cpp_qk_norm_rope_append(cpp, plain, nq, nkv, d, rot, norms):
    page, pages = 8, 24
    seq_ctx, q_lens = [19, 8, 70], [19, 1, 7]
    table, positions, seq_of_token, _, _ = paged(seq_ctx, q_lens, page, pages, 7, "cpu")
    T = sum(q_lens)
    qkv = rnd(T, (nq + 2 * nkv) * d, seed=8)
    qn = 1 + 0.1 * rnd(d, seed=9) if norms else None
    kn = 1 + 0.1 * rnd(d, seed=10) if norms else None
    inv_freq = torch.pow(torch.tensor(1e4), -2 * torch.arange(max(rot, 2) // 2, dtype=torch.float32) / max(rot, 2))
    outs = []
    for impl in (cpp, plain):
        q_out = torch.full((T, nq * d), float("nan"))
        kc = torch.full((pages, nkv, page, d), 7.0)
        vc = torch.full((pages, nkv, page, d), 7.0)
        impl.qk_norm_rope_append(qkv, q_out, kc, vc, qn, kn, inv_freq if rot else None, rot, 1e-6, 0.0,
                                 positions, seq_of_token, table, nq, nkv, d, page)
        outs.append((q_out, kc, vc))
    close(outs[0][0], outs[1][0], 3e-6, "q")
    close(outs[0][1], outs[1][1], 3e-6, "key cache")
    assert torch.equal(outs[0][2], outs[1][2]), "value cache"
    q_only = torch.empty(T, nq * d)
    cpp.qk_norm_rope_append(qkv[:, :nq * d].contiguous(), q_only, None, None, qn, kn, inv_freq if rot else None,
                            rot, 1e-6, 0.0, positions, seq_of_token, None, nq, nkv, d, page)
    close(q_only, outs[1][0], 3e-6, "q only")


@pytest.mark.parametrize("nq,nkv,d,window", [(4, 2, 16, None), (6, 3, 48, 24), (5, 1, 32, 7), (4, 4, 16, 1)])
def test_cpp_attention(cpp, plain, nq, nkv, d, window):
    page, pages = 8, 64
    seq_ctx, q_lens = [33, 64, 65, 16, 90], [33, 1, 1, 16, 21]
    table, positions, seq_of_token, q_start, ctx_len = paged(seq_ctx, q_lens, page, pages, 11, "cpu")
    T = sum(q_lens)
    q = rnd(T, nq * d, seed=12)
    kc, vc = fill_caches(table, seq_ctx, pages, nkv, page, d, "cpu")
    a, b = torch.empty(T, nq * d), torch.empty(T, nq * d)
    args = (table, q_start, ctx_len, seq_of_token, positions, nq, nkv, d, page, 1.0 / math.sqrt(d), window,
            max(q_lens), max(seq_ctx), min(q_lens))
    cpp.attention(q, kc, vc, a, *args)
    plain.attention(q, kc, vc, b, *args)
    close(a, b, 3e-6, "attention")


def test_cpp_sample(cpp, plain):
    vocab, R = 301, 40
    logits = rnd(R, vocab, seed=20, scale=2.0)
    logits[1, 17] = logits[1, 200] = 50.0                       # a tie: the lower id
    logits[2] = 0.0                                             # all equal: id 0
    a, b = torch.empty(R, dtype=torch.int32), torch.empty(R, dtype=torch.int32)
    cpp.sample(logits, None, None, a)
    plain.sample(logits, None, None, b)
    assert a.tolist() == b.tolist() and a[1] == 17 and a[2] == 0
    temps = torch.full((R,), 0.7)
    temps[0] = 0.0
    uni = torch.rand(R, generator=torch.Generator().manual_seed(22))
    uni[1], uni[2] = 0.0, 0.99999994
    cpp.sample(logits, temps, uni, a)
    plain.sample(logits, temps, uni, b)
    assert a[0] == int(logits[0].argmax())
    # the plain restatement rounds its probabilities to 32 bits first: allow the neighbour where u sits on an edge
    for r in range(R):
        if int(a[r]) != int(b[r]):
            p = torch.exp((logits[r].double() - logits[r].double().max()) / 0.7)
            cdf = torch.cumsum(p, 0) / p.sum()
            assert abs(int(a[r]) - int(b[r])) == 1 and abs(float(cdf[min(int(a[r]), int(b[r]))]) - float(uni[r])) < 1e-5


# ---------------------------------------------------------------- with a GPU: the kernels against C++

@pytest.fixture(scope="module")
def k():
    from chibillm_b200.kernels.ops import CudaKernels
    return CudaKernels(torch.device("cuda:0"))


DTYPES = [torch.float32, torch.bfloat16]


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
def test_kernels_against_cpp_elementwise(k, cpp, dtype):
    tol = 3e-6 if dtype == torch.float32 else 8e-3
    table = rnd(77, 88, seed=1, device="cuda", dtype=dtype)
    tokens = torch.tensor([0, 76, 7, 7, 31], dtype=torch.int32, device="cuda")
    a, b = torch.empty(5, 88, device="cuda"), torch.empty(5, 88, device="cuda")
    k.embed(tokens, table, a)
    cpp.embed(tokens, table, b)
    assert torch.equal(a, b)

    x = rnd(21, 200, seed=2, scale=3.0, device="cuda")
    w = (1 + 0.1 * rnd(200, seed=3, device="cuda")).to(dtype)
    a = torch.empty(21, 200, device="cuda", dtype=dtype)
    b = torch.empty_like(a)
    k.rmsnorm(x, w, 1e-5, 0.0, a)
    cpp.rmsnorm(x, w, 1e-5, 0.0, b)
    close(a, b, tol, "rmsnorm")

    gu = rnd(13, 2 * 176, seed=4, scale=3.0, device="cuda", dtype=dtype)
    a = torch.empty(13, 176, device="cuda", dtype=dtype)
    b = torch.empty_like(a)
    k.swiglu(gu, a)
    cpp.swiglu(gu, b)
    close(a, b, tol, "swiglu")

    rows = torch.tensor([12, 0, 7, 7], dtype=torch.int32, device="cuda")
    xs = rnd(13, 80, seed=5, device="cuda")
    a, b = torch.empty(4, 80, device="cuda"), torch.empty(4, 80, device="cuda")
    k.gather_rows(xs, rows, a)
    cpp.gather_rows(xs, rows, b)
    assert torch.equal(a, b)


@pytest.mark.gpu
@pytest.mark.parametrize("M", [3, 70, 200])
@pytest.mark.parametrize("dtype", DTYPES)
def test_kernels_against_cpp_linear(k, cpp, M, dtype):
    """The 32-bit product (CUDA cores) and the bfloat16 one (tcgen05: few rows, up to 128 rows, many rows)."""
    N, K = 136, 264
    x = rnd(M, K, seed=6, device="cuda", dtype=dtype)
    w = rnd(N, K, seed=7, scale=0.1, device="cuda", dtype=dtype)
    res = rnd(M, N, seed=8, device="cuda")
    a, b = res.clone(), res.clone()
    k.linear(x, w, a, residual=a)
    cpp.linear(x, w, b, residual=res)
    close(a, b, 3e-6 if dtype == torch.float32 else 2e-5, "linear onto the residual")
    a = torch.empty(M, N, device="cuda", dtype=dtype)
    b = torch.empty_like(a)
    k.linear(x, w, a)
    cpp.linear(x, w, b)
    k.check_error_word()
    close(a, b, 3e-6 if dtype == torch.float32 else 8e-3, "linear")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nq,nkv,d,rot,window", [(6, 2, 48, 48, None), (4, 4, 16, 8, 9), (5, 1, 128, 128, 40)])
def test_kernels_against_cpp_heads_and_attention(k, cpp, dtype, nq, nkv, d, rot, window):
    """Norm, rotation and the append into shuffled pages, then attention over those pages."""
    page, pages = 8, 48
    seq_ctx, q_lens = [19, 8, 70, 130], [19, 1, 7, 66]
    table, positions, seq_of_token, q_start, ctx_len = paged(seq_ctx, q_lens, page, pages, 7, "cuda")
    T = sum(q_lens)
    qkv = rnd(T, (nq + 2 * nkv) * d, seed=8, device="cuda", dtype=dtype)
    qn = (1 + 0.1 * rnd(d, seed=9, device="cuda")).to(dtype)
    kn = (1 + 0.1 * rnd(d, seed=10, device="cuda")).to(dtype)
    inv_freq = torch.pow(torch.tensor(1e4), -2 * torch.arange(rot // 2, dtype=torch.float32) / rot).cuda()
    kc0, vc0 = fill_caches(table, seq_ctx, pages, nkv, page, d, "cuda", dtype, other=7.0)
    tol = 3e-6 if dtype == torch.float32 else 8e-3
    outs = []
    for impl in (k, cpp):
        q_out = torch.full((T, nq * d), float("nan"), dtype=dtype, device="cuda")
        kc, vc = kc0.clone(), vc0.clone()
        impl.qk_norm_rope_append(qkv, q_out, kc, vc, qn, kn, inv_freq, rot, 1e-6, 0.0, positions, seq_of_token,
                                 table, nq, nkv, d, page)
        outs.append((q_out, kc, vc))
    k.check_error_word()
    close(outs[0][0], outs[1][0], tol, "q")
    close(outs[0][1], outs[1][1], tol, "key cache")
    assert torch.equal(outs[0][2], outs[1][2]), "value cache"
    q, kc, vc = outs[1]
    a = torch.full((T, nq * d), float("nan"), dtype=dtype, device="cuda")
    b = torch.empty_like(a)
    args = (table, q_start, ctx_len, seq_of_token, positions, nq, nkv, d, page, 1.0 / math.sqrt(d), window,
            max(q_lens), max(seq_ctx), min(q_lens))
    k.attention(q, kc, vc, a, *args)
    cpp.attention(q, kc, vc, b, *args)
    k.check_error_word()
    close(a, b, 1e-5 if dtype == torch.float32 else 1.2e-2, "attention")


@pytest.mark.gpu
def test_kernels_against_cpp_sample(k, cpp):
    vocab, R = 1003, 48
    logits = rnd(R, vocab, seed=20, scale=2.0, device="cuda")
    logits[1, 17] = logits[1, 200] = 50.0
    logits[2] = 0.0
    a = torch.empty(R, dtype=torch.int32, device="cuda")
    b = torch.empty_like(a)
    k.sample(logits, None, None, a)
    cpp.sample(logits, None, None, b)
    assert a.tolist() == b.tolist()
    temps = torch.full((R,), 0.8, device="cuda")
    temps[0] = 0.0
    uni = torch.rand(R, generator=torch.Generator().manual_seed(22)).cuda()
    k.sample(logits, temps, uni, a)
    cpp.sample(logits, temps, uni, b)
    differ = [r for r in range(R) if int(a[r]) != int(b[r])]
    for r in differ:                 # 32-bit sums on the device: a neighbour, and only where u sits on an edge
        p = torch.exp((logits[r].double() - logits[r].double().max()) / 0.8)
        cdf = (torch.cumsum(p, 0) / p.sum()).cpu()
        edge = float(cdf[min(int(a[r]), int(b[r]))])
        assert abs(int(a[r]) - int(b[r])) == 1 and abs(edge - float(uni[r])) < 1e-4, f"row {r}"
    assert len(differ) <= 2
