"""How the many-row matrix product cuts its output (``many_rows_plan`` in
chibillm_b200/csrc/gemm_tcgen05.cu), asked of the built kernel library without a GPU:
the answer depends on the shape and the number of SMs only (148 where no device says otherwise).
Each expectation below is a measured best among the forced variants on a B200."""
import ctypes
import os

import pytest

from chibillm_b200.csrc import build


@pytest.fixture(scope="module")
def plan():
    path = build.library_path("chibi_kernels")
    if not os.path.isfile(path):
        pytest.skip("the kernel library is not built here")
    lib = ctypes.CDLL(path)
    lib.chibi_gemm_many_rows_plan.restype = ctypes.c_int
    lib.chibi_gemm_many_rows_plan.argtypes = [ctypes.c_int] * 3
    lib.chibi_gemm_set_pair_tiles.argtypes = [ctypes.c_int] * 2
    lib.chibi_gemm_set_pair_tiles(1, 256)
    return lambda m, n, k: lib.chibi_gemm_many_rows_plan(m, n, k)


SINGLE_256, SINGLE_128, PAIRS_256, PAIRS_128 = 256, 128, 257, 129


@pytest.mark.parametrize("m,n,k,expected", [
    # a prompt of 2,048 tokens at the Qwen3-8B sizes: all four products by pairs on 256 x 256
    (2048, 6144, 4096, PAIRS_256), (2048, 4096, 4096, PAIRS_256), (2048, 24576, 4096, PAIRS_256),
    (2048, 4096, 12288, PAIRS_256),
    # 1,024 rows of q|k|v: 96 tiles of 256 x 256 fill 74 pairs badly, 192 of 256 x 128 better
    (1024, 6144, 4096, PAIRS_128),
    # 512 rows of o: 64 tiles of 256 columns, or 128 of 128 by pairs
    (512, 4096, 4096, PAIRS_128),
    # 384 rows: two blocks of 256 would be a quarter empty, three of 128 are full; 448 rows fill both alike
    (384, 24576, 4096, SINGLE_256), (448, 24576, 4096, PAIRS_256),
    # Qwen3-14B down at 2,048 rows: a last round of 24 tiles, K long: shared out by single CTAs
    (2048, 5120, 17408, SINGLE_256),
    # the same tiles with K short: adding the shared-out round up would cost more than pairs lose
    # (measured: 94.2 us shared out, 88.1 by pairs on 256 x 256, 86.0 on 256 x 128)
    (2048, 5120, 5120, PAIRS_128),
    # 4,096 x 6,144: a last round of 28 single tiles against six rounds of pairs
    (4096, 6144, 4096, PAIRS_256),
    # columns that are no multiple of 256, of 128
    (2048, 896, 4096, SINGLE_128), (2048, 1000, 4096, 0),
])
def test_plan_of_measured_shapes(plan, m, n, k, expected):
    assert plan(m, n, k) == expected


def test_plan_never_pairs_below_256_rows(plan):
    for n, k in ((4096, 4096), (6144, 4096), (24576, 4096), (4096, 12288), (1024, 3072)):
        for m in (129, 160, 200, 255):
            assert plan(m, n, k) in (SINGLE_256, SINGLE_128)
