"""Pins the CPU oracle (oracle/oracle_blas.c) to the reference: bit-identical to the reference's
own NaiveBlas code where that was compiled (oracle/_ref), bit-identical to the committed golden
outputs everywhere, equal to the reference's known-answer tests and fixed sample inputs, and
within rounding of a Netlib-interface BLAS (the reference test-suite's own oracle interface,
src/tests/correctness/blas-lapack.c:70, :124)."""
import os

import numpy as np
import pytest

import oracle
from oracle import ColumnMajor, Left, Lower, NonUnit, NoTrans, Right, RowMajor, Trans, Unit, Upper
from tests import cases

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "level3_golden.npz")


@pytest.fixture(scope="module")
def golden():
    return np.load(GOLDEN)


def run_gemm(c, impl):
    A, B, C = cases.gemm_buffers(c)
    oracle.gemm(c["order"], c["transA"], c["transB"], c["M"], c["N"], c["K"], c["alpha"], A, c["offA"], c["lda"],
                B, c["offB"], c["ldb"], c["beta"], C, c["offC"], c["ldc"], impl=impl)
    return C


def run_trsm(c, impl):
    A, B = cases.trsm_buffers(c)
    oracle.trsm(c["order"], c["side"], c["uplo"], c["transA"], c["diag"], c["M"], c["N"], c["alpha"], A, c["offA"],
                c["lda"], B, c["offB"], c["ldb"], impl=impl)
    return B


def same_bits(a, b):
    return a.shape == b.shape and np.array_equal(a.view(np.uint8), b.view(np.uint8))


def test_port_matches_golden_gemm(built_oracle, golden):
    for name, c in cases.golden_gemm_cases().items():
        assert same_bits(run_gemm(c, "port"), golden[name]), name


def test_port_matches_golden_trsm(built_oracle, golden):
    for name, c in cases.golden_trsm_cases().items():
        assert same_bits(run_trsm(c, "port"), golden[name]), name


@pytest.mark.skipif(not oracle.have_ref(), reason="reference's own naive_blas.cpp was not compiled here")
def test_port_matches_reference_code(built_oracle):
    """Wider sweep than the golden file: port and reference code must agree to the bit."""
    n = 0
    for prec in "sd":
        for c in cases.sweep_gemm_cases(prec, "uniform")[::3]:
            assert same_bits(run_gemm(c, "port"), run_gemm(c, "ref")), c
            n += 1
        for c in cases.sweep_trsm_cases(prec)[::5]:
            if max(c["M"], c["N"]) > 140:
                continue
            assert same_bits(run_trsm(c, "port"), run_trsm(c, "ref")), c
            n += 1
    assert n > 100


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
def test_trsm_known_answer(built_oracle, dtype):
    """TRSM_extratest of the reference (src/tests/correctness/corr-trsm.cpp:240-452): column-major,
    Left/Upper/NoTrans/NonUnit, M=5, N=2, lda=ldb=32; A has j+1 on the diagonal, ones above, zeros
    below; B(row j) = T(M) - T(j+1) + (j+1)^2 with T(n) = n(n+1)/2.  The exact solution is X(row j) = j+1."""
    M, N, ld = 5, 2, 32
    A = np.zeros(M * ld, dtype=dtype)
    B = np.zeros(N * ld, dtype=dtype)
    tri = lambda n: n * (n + 1) // 2
    for col in range(M):
        for row in range(M):
            A[col * ld + row] = (row + 1) if row == col else (0.0 if row > col else 1.0)
    for col in range(N):
        for row in range(M):
            B[col * ld + row] = tri(M) - tri(row + 1) + (row + 1) ** 2
    oracle.trsm(ColumnMajor, Left, Upper, NoTrans, NonUnit, M, N, 1.0, A, 0, ld, B, 0, ld)
    X = oracle.view(B, ColumnMajor, NoTrans, M, N, ld, 0)
    expect = np.arange(1, M + 1, dtype=dtype)[:, None].repeat(N, axis=1)
    assert np.max(np.abs(X - expect)) <= 1e-5          # ETST_TOLERENCE of the reference test
    assert np.all(B.reshape(N, ld)[:, M:] == 0)          # padding rows untouched


def test_sample_sgemm_inputs(built_oracle):
    """Fixed inputs of src/samples/example_sgemm.c:32-71 (row-major, M-1 x N-1 x K-1 sub-problem at
    offsets K+1 / N+1 / N+1, alpha 10, beta 20); all values are small integers so the result is exact."""
    M, N, K = 4, 3, 5
    A = np.array([[10 * (i + 1) + (j + 1) for j in range(K)] for i in range(M)], dtype=np.float32)
    B = np.array([[10 * (i + 1) + (j + 1) for j in range(N)] for i in range(K)], dtype=np.float32)
    C = np.array([[10 * (i + 1) + (j + 1) for j in range(N)] for i in range(M)], dtype=np.float32)
    Cb = C.ravel().copy()
    oracle.gemm(RowMajor, NoTrans, NoTrans, M - 1, N - 1, K - 1, 10.0, A.ravel(), K + 1, K, B.ravel(), N + 1, N,
                20.0, Cb, N + 1, N)
    expect = C.copy()
    expect[1:, 1:] = 10.0 * (A[1:, 1:].astype(np.float64) @ B[1:, 1:].astype(np.float64)) + 20.0 * C[1:, 1:]
    assert np.array_equal(Cb.reshape(M, N), expect.astype(np.float32))


def test_sample_strsm_inputs(built_oracle):
    """Fixed inputs of src/samples/example_strsm.c:31-60 (row-major Left/Upper/NoTrans/NonUnit,
    (M-1) x (N-1) sub-problem at offsets M+1 / N+1, alpha 10)."""
    M, N = 4, 5
    A = np.array([[11, 12, 13, 14], [0, 22, 23, 24], [0, 0, 33, 34], [0, 0, 0, 44]], dtype=np.float32)
    B = np.array([[10 * (i + 1) + (j + 1) for j in range(N)] for i in range(M)], dtype=np.float32)
    Bb = B.ravel().copy()
    oracle.trsm(RowMajor, Left, Upper, NoTrans, NonUnit, M - 1, N - 1, 10.0, A.ravel(), M + 1, M, Bb, N + 1, N)
    X = Bb.reshape(M, N)[1:, 1:].astype(np.float64)
    resid = A[1:, 1:].astype(np.float64) @ X - 10.0 * B[1:, 1:]
    assert np.max(np.abs(resid)) < 1e-3
    assert np.array_equal(Bb.reshape(M, N)[0, :], B[0, :]) and np.array_equal(Bb.reshape(M, N)[:, 0], B[:, 0])


@pytest.mark.parametrize("prec", ["s", "d"])
def test_oracle_vs_netlib_interface(built_oracle, prec):
    """scipy's BLAS (Netlib interface, the kind of library the reference suite links as its oracle)
    agrees with the port within the stated tolerances."""
    from scipy.linalg import blas
    dt = cases.DT[prec]
    c = cases.gemm_case(prec, ColumnMajor, Trans, NoTrans, 65, 33, 129, alpha=1.5, beta=0.5)
    opA, opB, C = cases.gemm_logical(c)
    got = run_gemm(c, "port")
    Cg = oracle.view(got, ColumnMajor, NoTrans, 65, 33, c["ldc"], 0)
    f = blas.sgemm if prec == "s" else blas.dgemm
    ref = f(1.5, np.asfortranarray(opA.T), np.asfortranarray(opB), beta=0.5, c=np.asfortranarray(C), trans_a=1)
    assert np.allclose(Cg, ref, rtol=0, atol=4 * 129 * oracle.unit_roundoff(dt) * 129 * 2)
    assert oracle.gemm_error_ratio(Cg, 1.5, opA, opB, 0.5, C, 129, dt) <= 1.0

    t = cases.trsm_case(prec, ColumnMajor, Left, Lower, NoTrans, NonUnit, 64, 19, alpha=2.0)
    A, B = cases.trsm_logical(t)
    Bb = run_trsm(t, "port")
    X = oracle.view(Bb, ColumnMajor, NoTrans, 64, 19, t["ldb"], 0)
    g = blas.strsm if prec == "s" else blas.dtrsm
    ref = g(2.0, np.asfortranarray(np.nan_to_num(A)), np.asfortranarray(B), side=0, lower=1, trans_a=0, diag=0)
    assert np.allclose(X, ref, rtol=1e-4 if prec == "s" else 1e-12)
    assert oracle.trsm_backward_ratio(X, 2.0, cases.trsm_op_triangle(t, A), B, Left, dt) <= 1.0


def test_poison_outside_triangle_never_read(built_oracle):
    """The NaN outside the referenced triangle (and on a unit diagonal) must not reach the result."""
    for c in cases.sweep_trsm_cases("d")[::7]:
        if max(c["M"], c["N"]) > 140:
            continue
        A, B = cases.trsm_logical(c)
        Bb = run_trsm(c, "port")
        X = oracle.view(Bb, c["order"], NoTrans, c["M"], c["N"], c["ldb"], c["offB"])
        assert np.all(np.isfinite(X)), c
        assert oracle.trsm_backward_ratio(X, c["alpha"], cases.trsm_op_triangle(c, A), B, c["side"], np.float64) <= 1.0, c


def test_trsm_delta_bound_accepts_a_netlib_solution(built_oracle):
    """The restated acceptance rule of the reference's TRSM tests (trsmDelta, src/tests/correctness/trsm-delta.h:44-240):
    the oracle's solution and a Netlib-interface solution (what the reference's tests compare the library against)
    must lie within delta of each other on reference-style inputs, for both sides, both triangles, both precisions --
    and delta must mean something: for a typical entry it is a small fraction of the solution (it is a loose bound:
    a few per cent in float at order 150, because it adds the absolute errors of a whole column)."""
    from scipy.linalg import blas
    import oracle
    from oracle import ColumnMajor, Left, Right, Lower, Upper, NoTrans, Trans, NonUnit, Unit
    for dt, fn in ((np.float32, blas.strsm), (np.float64, blas.dtrsm)):
        for side, uplo, trans, diag in ((Left, Lower, NoTrans, NonUnit), (Left, Upper, Trans, Unit), (Right, Upper, NoTrans, NonUnit),
                                        (Right, Lower, Trans, NonUnit)):
            M, N = (150, 40) if side == Left else (40, 150)
            n = M if side == Left else N
            A, B = oracle.trsm_inputs(n, (M, N), uplo, diag, dt, seed=77, poison=False)
            T = oracle.clean_triangle(A, uplo, diag)
            ld = n
            Ab = oracle.pack(A, ColumnMajor, NoTrans, ld, 0)
            Bb = oracle.pack(B, ColumnMajor, NoTrans, M, 0)
            oracle.trsm(ColumnMajor, side, uplo, trans, diag, M, N, 1.5, Ab, 0, ld, Bb, 0, M)
            X = oracle.view(Bb, ColumnMajor, NoTrans, M, N, M, 0)
            Xn = fn(dt(1.5), np.asfortranarray(T), np.asfortranarray(B), side=1 if side == Right else 0, lower=1 if uplo == Lower else 0,
                    trans_a=1 if trans == Trans else 0, diag=1 if diag == Unit else 0)
            delta = oracle.trsm_delta(side, uplo, trans, diag, T, B, 1.5, dt)
            assert delta.shape == (M, N) and np.all(delta > 0)
            assert np.all(np.abs(X.astype(np.float64) - Xn.astype(np.float64)) <= delta)
            assert np.median(delta / (np.abs(Xn) + 1e-30)) < (0.1 if dt == np.float32 else 1e-9)
