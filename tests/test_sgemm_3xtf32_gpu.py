"""The optional tcgen05 SGEMM variant (3xTF32 operand split, clblasB200SetGemmPath(4)).

It is not an FFMA evaluation, so it is qualified the way the stated tolerance demands and NOT with
the exact-integer inputs (small integers fit a TF32 mantissa and would hide the split): real-valued
inputs, max |C - C_exact| / (|alpha||A||B| + |beta||C|) <= 4*K*u with u = 2^-24, on every transpose
case, ragged shapes, unaligned operands, and the benchmark's SGEMM shapes at reduced K."""
import numpy as np
import pytest

import oracle
from oracle import ColumnMajor, NoTrans, RowMajor, Trans
from tests import cases
from tests.gpu_util import outside_untouched, run_gemm_gpu

pytestmark = pytest.mark.gpu

PATH_3XTF32 = 4


@pytest.fixture()
def tf32_path(lib):
    old = lib.set_gemm_path(PATH_3XTF32)
    yield lib
    lib.set_gemm_path(old)


def _check(lib, c):
    logical = cases.gemm_logical(c)
    bufs = cases.gemm_buffers(c, logical)
    st, got = run_gemm_gpu(lib, c, bufs)
    assert st == lib.clblasSuccess, lib.STATUS_NAME.get(st, st)
    assert lib.last_gemm_kernel() == "sgemm_3xtf32_tcgen05", lib.last_gemm_kernel()
    assert outside_untouched(bufs[2], got, c)
    Cg = oracle.view(got, c["order"], NoTrans, c["M"], c["N"], c["ldc"], c["offC"])
    assert np.all(np.isfinite(Cg))
    opA, opB, C = logical
    ratio = oracle.gemm_error_ratio(Cg, c["alpha"], opA, opB, c["beta"], C, c["K"], np.float32)
    assert ratio <= 1.0, (ratio, c)
    return ratio


def test_native_layout_small(tf32_path):
    """A stored K x M, B stored K x N (the kernel's native layout), one and several tiles, ragged K."""
    for M, N, K in ((128, 256, 32), (128, 256, 64), (256, 512, 160), (130, 300, 77), (64, 40, 200), (1, 1, 9)):
        c = cases.gemm_case("s", ColumnMajor, Trans, NoTrans, M, N, K, alpha=1.0, beta=0.0, seed=41 + M)
        for k in ("lda", "ldb", "ldc"):
            c[k] = (c[k] + 3) // 4 * 4
        _check(tf32_path, c)
    assert tf32_path.device_fault() == 0


def test_all_transposes_and_orders(tf32_path):
    worst = 0.0
    seed = 500
    for order in (ColumnMajor, RowMajor):
        for ta in (NoTrans, Trans):
            for tb in (NoTrans, Trans):
                seed += 1
                c = cases.gemm_case("s", order, ta, tb, 515, 389, 1031, alpha=1.5, beta=0.5, pad=(3, 1, 2), off=(1, 2, 3),
                                    seed=seed)
                worst = max(worst, _check(tf32_path, c))
                seed += 1
                c = cases.gemm_case("s", order, ta, tb, 1024, 768, 2048, alpha=-2.0, beta=0.25, mode="normal", seed=seed)
                worst = max(worst, _check(tf32_path, c))
    assert worst <= 1.0
    assert tf32_path.device_fault() == 0


def test_split_recovers_fp32_accuracy(tf32_path):
    """The point of the split: the error must sit near FP32 rounding, far below what one TF32 product
    would give (relative 2^-11).  Measured against |A||B| it has to stay under 2^-19 even for K = 8."""
    c = cases.gemm_case("s", ColumnMajor, Trans, NoTrans, 256, 256, 8, alpha=1.0, beta=0.0, seed=77)
    opA, opB, C = cases.gemm_logical(c)
    st, got = run_gemm_gpu(tf32_path, c, cases.gemm_buffers(c, (opA, opB, C)))
    assert st == tf32_path.clblasSuccess
    Cg = oracle.view(got, ColumnMajor, NoTrans, 256, 256, c["ldc"], 0).astype(np.float64)
    A64, B64 = opA.astype(np.float64), opB.astype(np.float64)
    err = np.abs(Cg - A64 @ B64) / (np.abs(A64) @ np.abs(B64))
    assert err.max() <= 2.0 ** -19, err.max()
