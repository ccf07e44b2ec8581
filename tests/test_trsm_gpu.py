"""TRSM parity on the GPU, through the C ABI, against the CPU oracle.

Inputs follow the reference's generator (src/tests/include/blas-random.h:175-342): diagonally
dominant triangles with NaN outside the referenced triangle and on a unit diagonal, so that an
illegal read poisons the result.  Acceptance: entrywise backward error
|alpha B - op(A) X| / (|op(A)||X| + |alpha||B|) <= 4*M*u, plus agreement with the oracle's solution
within the forward bound that backward error implies for these well-conditioned systems."""
import numpy as np
import pytest

import oracle
from oracle import ColumnMajor, Left, Lower, NonUnit, NoTrans, Right, RowMajor, Trans, Unit, Upper
from tests import cases
from tests.gpu_util import outside_untouched, run_trsm_gpu, run_trsm_oracle

pytestmark = pytest.mark.gpu


def check_trsm(cb, c):
    logical = cases.trsm_logical(c)
    bufs = cases.trsm_buffers(c, logical)
    before = bufs[1].copy()
    st, got = run_trsm_gpu(cb, c, bufs)
    assert st == cb.clblasSuccess, (cb.STATUS_NAME.get(st, st), c)
    assert outside_untouched(before, got, c), c
    dt = cases.DT[c["prec"]]
    X = oracle.view(got, c["order"], NoTrans, c["M"], c["N"], c["ldb"], c["offB"])
    assert np.all(np.isfinite(X)), c
    A, B = logical
    T = cases.trsm_op_triangle(c, A)
    ratio = oracle.trsm_backward_ratio(X, c["alpha"], T, B, c["side"], dt)
    assert ratio <= 1.0, (ratio, c)
    want = run_trsm_oracle(c, bufs)
    Xo = oracle.view(want, c["order"], NoTrans, c["M"], c["N"], c["ldb"], c["offB"])
    n = T.shape[0]
    scale = np.max(np.abs(Xo)) + 1e-30
    assert np.max(np.abs(X - Xo)) / scale <= 64 * n * oracle.unit_roundoff(dt), c
    return ratio


@pytest.mark.parametrize("prec", ["s", "d"])
def test_sweep_all_variants(lib, prec):
    """order x side x uplo x trans (incl. ConjTrans) x diag, sizes below/at/above the 128 block."""
    for c in cases.sweep_trsm_cases(prec):
        check_trsm(lib, c)


@pytest.mark.parametrize("prec", ["s", "d"])
def test_known_answer(lib, prec):
    """TRSM_extratest of the reference (src/tests/correctness/corr-trsm.cpp:240-452): exact solution
    X(row j) = j+1, lda = ldb = 32 != M, padding rows must stay zero; tolerance 1e-5 as there."""
    import torch
    dt = cases.DT[prec]
    M, N, ld = 5, 2, 32
    A = np.zeros(M * ld, dtype=dt)
    B = np.zeros(N * ld, dtype=dt)
    tri = lambda n: n * (n + 1) // 2
    for col in range(M):
        for row in range(M):
            A[col * ld + row] = (row + 1) if row == col else (0.0 if row > col else 1.0)
    for col in range(N):
        for row in range(M):
            B[col * ld + row] = tri(M) - tri(row + 1) + (row + 1) ** 2
    c = dict(kind="trsm", prec=prec, order=ColumnMajor, side=Left, uplo=Upper, transA=NoTrans, diag=NonUnit, M=M, N=N,
             alpha=1.0, lda=ld, ldb=ld, offA=0, offB=0)
    st, got = run_trsm_gpu(lib, c, (A, B))
    assert st == lib.clblasSuccess
    want = run_trsm_oracle(c, (A, B))
    assert np.max(np.abs(got - want)) <= 1e-5
    X = got.reshape(N, ld)
    assert np.max(np.abs(X[:, :M] - np.arange(1, M + 1))) <= 1e-5
    assert np.all(X[:, M:] == 0)


@pytest.mark.parametrize("prec", ["s", "d"])
def test_alpha_zero(lib, prec):
    c = cases.trsm_case(prec, ColumnMajor, Left, Lower, NoTrans, NonUnit, 70, 33, alpha=0.0, pad=(0, 5))
    A, B = cases.trsm_logical(c)
    bufs = cases.trsm_buffers(c, (A * np.nan, B))
    st, got = run_trsm_gpu(lib, c, bufs)
    assert st == lib.clblasSuccess
    assert np.all(oracle.view(got, ColumnMajor, NoTrans, 70, 33, c["ldb"], 0) == 0)
    assert outside_untouched(bufs[1], got, c)


def test_medium_dtrsm_left_lower(lib):
    """The benchmark's DTRSM (Left/Lower/NoTrans/NonUnit) at a size the CPU check finishes quickly: 1024 x 1024
    lower triangle (diag U[1,2], strict lower U[-1,1]/n, garbage above), 512 right-hand sides."""
    n, nrhs = 1024, 512
    g = oracle.rng(12345, 21)
    A = np.tril(g.uniform(-1, 1, (n, n)) / n, -1) + np.diag(g.uniform(1, 2, n))
    A[np.triu(np.ones((n, n), dtype=bool), 1)] = np.nan
    A[0, n - 1] = 1e300
    B = g.standard_normal((n, nrhs))
    c = cases.trsm_case("d", ColumnMajor, Left, Lower, NoTrans, NonUnit, n, nrhs)
    bufs = cases.trsm_buffers(c, (A, B))
    st, got = run_trsm_gpu(lib, c, bufs)
    assert st == lib.clblasSuccess
    X = oracle.view(got, ColumnMajor, NoTrans, n, nrhs, n, 0)
    assert oracle.trsm_backward_ratio(X, 1.0, np.tril(np.nan_to_num(A, nan=0.0, posinf=0.0)) * (np.tril(np.ones((n, n))) > 0), B, Left, np.float64) <= 1.0
