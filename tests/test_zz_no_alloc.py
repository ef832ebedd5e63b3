"""The allocation-free matrix product, called through its exported C symbol.

Some callers of this library cannot allocate device memory at all -- a plug-in
whose host application owns the device heap, or a loop that has promised not to
call cudaMalloc after start-up.  For them ``chibi_gemm_bf16_noalloc`` keeps the
split-K partial sums in an array that is built into the library instead of in a
scratch array that the caller would have to provide.  The test calls it twice in
a row (the array keeps the first call's contents; the second result must not
care) and compares with the ordinary entry point, which gets its scratch from
torch.  This file is collected last, so a run that stops at the first failure
has run every other test before it.
"""
import ctypes
from ctypes import c_int, c_longlong, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu

NOALLOC_SCRATCH_FLOATS = 1 << 20
ERR_SCRATCH_LIMIT = -4


@pytest.fixture(scope="module")
def lib():
    from chibillm_b200.csrc import build
    handle = ctypes.CDLL(build.ensure_library("chibi_kernels"))
    P, I, L = c_void_p, c_int, c_longlong
    handle.chibi_gemm_bf16_noalloc.argtypes = [P, P, P, I, P, I, I, I, L, L, L, L, P, P]
    handle.chibi_gemm_bf16_noalloc.restype = c_int
    handle.chibi_gemm_bf16.argtypes = [P, P, P, I, P, I, I, I, L, L, L, L, P, L, P, P]
    handle.chibi_gemm_bf16.restype = c_int
    handle.chibi_gemm_bf16_splits.argtypes = [I, I, I]
    handle.chibi_gemm_bf16_splits.restype = c_int
    handle.chibi_error_string.argtypes = [I]
    handle.chibi_error_string.restype = ctypes.c_char_p
    return handle


def _inputs(M, N, K, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(M, K, generator=g, device="cuda").to(torch.bfloat16)
    w = (0.05 * torch.randn(N, K, generator=g, device="cuda")).to(torch.bfloat16)
    res = torch.randn(M, N, generator=g, device="cuda")
    return x, w, res


def test_two_calls_in_a_row_match_the_ordinary_entry_point(lib):
    stream = torch.cuda.current_stream().cuda_stream
    error = torch.zeros(1, dtype=torch.int32, device="cuda")
    # (8, 4096, 4096) splits the K range ten ways; the second call is smaller, so
    # most of the array still holds the first call's partial sums
    for seed, (M, N, K) in enumerate([(8, 4096, 4096), (3, 1000, 2048)]):
        splits = lib.chibi_gemm_bf16_splits(M, N, K)
        assert splits > 1 and splits * M * N <= NOALLOC_SCRATCH_FLOATS
        x, w, res = _inputs(M, N, K, seed)
        for out_type, dtype in ((0, torch.float32), (1, torch.bfloat16)):
            residual = res if out_type == 0 else None
            got = torch.full((M, N), float("nan"), dtype=dtype, device="cuda")
            status = lib.chibi_gemm_bf16_noalloc(
                x.data_ptr(), w.data_ptr(), got.data_ptr(), out_type,
                residual.data_ptr() if residual is not None else None, M, N, K, K, K, N, N,
                error.data_ptr(), stream)
            assert status == 0, lib.chibi_error_string(status).decode()
            expected = torch.full((M, N), float("nan"), dtype=dtype, device="cuda")
            scratch = torch.empty(splits * M * N, dtype=torch.float32, device="cuda")
            status = lib.chibi_gemm_bf16(
                x.data_ptr(), w.data_ptr(), expected.data_ptr(), out_type,
                residual.data_ptr() if residual is not None else None, M, N, K, K, K, N, N,
                scratch.data_ptr(), scratch.numel(), error.data_ptr(), stream)
            assert status == 0
            torch.cuda.synchronize()
            plain = x.float() @ w.float().t() + (residual if residual is not None else 0)
            scale = float(plain.abs().max())
            tol = 2e-5 if dtype == torch.float32 else 8e-3
            assert float((got.float() - expected.float()).abs().max()) <= tol * scale
            assert float((got.float() - plain).abs().max()) <= tol * scale
    assert int(error.item()) == 0


def test_the_call_allocates_nothing_and_forgets_the_call_before(lib):
    """Free device memory is the same before and after warmed calls, and a call
    that does not split K (more than 128 rows) right after one that does gives
    the result of a call on its own: nothing of the array's old contents is read."""
    stream = torch.cuda.current_stream().cuda_stream
    error = torch.zeros(1, dtype=torch.int32, device="cuda")
    shapes = [(8, 4096, 4096), (5, 1024, 8192), (160, 512, 1024)]
    assert lib.chibi_gemm_bf16_splits(*shapes[0]) != lib.chibi_gemm_bf16_splits(*shapes[1]) > 1
    assert lib.chibi_gemm_bf16_splits(*shapes[2]) == 1
    cases = []
    for seed, (M, N, K) in enumerate(shapes):
        x, w, _ = _inputs(M, N, K, 20 + seed)
        cases.append((M, N, K, x, w, torch.empty(M, N, dtype=torch.float32, device="cuda")))

    def call(case):
        M, N, K, x, w, out = case
        out.fill_(float("nan"))
        status = lib.chibi_gemm_bf16_noalloc(x.data_ptr(), w.data_ptr(), out.data_ptr(), 0, None, M, N, K,
                                             K, K, N, 0, error.data_ptr(), stream)
        assert status == 0, lib.chibi_error_string(status).decode()

    for case in cases:                      # warm: kernel images, attributes, the array's address
        call(case)
    torch.cuda.synchronize()
    alone = []
    for case in cases:
        call(case)
        torch.cuda.synchronize()
        alone.append(case[5].clone())
    free_before, _ = torch.cuda.mem_get_info()
    for order in ((0, 1, 2), (1, 0, 2), (2, 1, 0)):
        for i in order:
            call(cases[i])
            torch.cuda.synchronize()
            assert torch.equal(cases[i][5], alone[i]), f"shape {shapes[i]} after another call"
            plain = cases[i][3].float() @ cases[i][4].float().t()
            assert float((cases[i][5] - plain).abs().max()) <= 2e-5 * float(plain.abs().max())
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before, "device memory was allocated or freed by the calls"
    assert int(error.item()) == 0


def test_a_product_beyond_the_built_in_scratch_is_refused(lib):
    M, N, K = 32, 4096, 12288
    splits = lib.chibi_gemm_bf16_splits(M, N, K)
    assert splits * M * N > NOALLOC_SCRATCH_FLOATS
    x, w, _ = _inputs(M, N, K, 5)
    out = torch.zeros(M, N, dtype=torch.float32, device="cuda")
    status = lib.chibi_gemm_bf16_noalloc(x.data_ptr(), w.data_ptr(), out.data_ptr(), 0, None, M, N, K,
                                         K, K, N, 0, None, torch.cuda.current_stream().cuda_stream)
    assert status == ERR_SCRATCH_LIMIT
    assert b"scratch" in lib.chibi_error_string(status)
    torch.cuda.synchronize()
    assert float(out.abs().max()) == 0.0        # nothing was launched
