"""GEMM on host matrices (clblasB200SgemmHost / clblasB200DgemmHost): the pipelined upload / multiply / download
must give exactly what the device routine gives on integer inputs, for every order and transposition, with padded
leading dimensions and offsets, across several column blocks and K-slabs; padding of the host C keeps its bits."""
import numpy as np
import pytest
import torch

import oracle
from oracle import ColumnMajor, NoTrans, RowMajor, Trans
from tests import cases
from tests.gpu_util import same_bits

pytestmark = pytest.mark.gpu


def run_host(cb, c, bufs):
    A, B, C = (torch.from_numpy(x).pin_memory() for x in bufs)
    fn = cb.clblasB200SgemmHost if c["prec"] == "s" else cb.clblasB200DgemmHost
    st = fn(c["order"], c["transA"], c["transB"], c["M"], c["N"], c["K"], c["alpha"], A, c["offA"], c["lda"],
            B, c["offB"], c["ldb"], c["beta"], C, c["offC"], c["ldc"])
    torch.cuda.synchronize()
    return st, C.numpy().copy()


@pytest.mark.parametrize("prec", ["s", "d"])
def test_small_cases_equal_the_oracle(lib, prec):
    for c in cases.sweep_gemm_cases(prec, "int")[::3]:
        bufs = cases.gemm_buffers(c)
        st, got = run_host(lib, c, bufs)
        assert st == lib.clblasSuccess, (lib.STATUS_NAME.get(st, st), c)
        want = bufs[2].copy()
        oracle.gemm(c["order"], c["transA"], c["transB"], c["M"], c["N"], c["K"], c["alpha"], bufs[0], c["offA"], c["lda"],
                    bufs[1], c["offB"], c["ldb"], c["beta"], want, c["offC"], c["ldc"])
        assert np.array_equal(got, want, equal_nan=True), c
        mask = oracle.outside_mask(got.size, c["order"], NoTrans, c["M"], c["N"], c["ldc"], c["offC"])
        assert same_bits(got[mask], bufs[2][mask]), c


@pytest.mark.parametrize("prec,order,ta,tb", [("d", ColumnMajor, Trans, NoTrans), ("s", ColumnMajor, NoTrans, Trans),
                                               ("d", RowMajor, NoTrans, NoTrans), ("s", RowMajor, Trans, Trans)])
def test_several_blocks_and_slabs(lib, prec, order, ta, tb):
    """8192 x 4200 x 2100: two K-slabs and (column-major) three column blocks of C."""
    M, N, K = (8192, 4200, 2100) if order == ColumnMajor else (4200, 8192, 2100)
    c = cases.gemm_case(prec, order, ta, tb, M, N, K, alpha=2.0, beta=-1.0, pad=(3, 1, 2), off=(5, 2, 7), mode="int", seed=77)
    g = oracle.rng(77, 5)
    dt = cases.DT[prec]
    logical = (g.integers(-3, 4, (M, K)).astype(dt), g.integers(-3, 4, (K, N)).astype(dt), g.integers(-3, 4, (M, N)).astype(dt))
    bufs = cases.gemm_buffers(c, logical)
    st, got = run_host(lib, c, bufs)
    assert st == lib.clblasSuccess
    want = 2.0 * (logical[0].astype(np.float64) @ logical[1].astype(np.float64)) - logical[2]
    X = oracle.view(got, order, NoTrans, M, N, c["ldc"], c["offC"])
    assert np.array_equal(X.astype(np.float64), want)
    mask = oracle.outside_mask(got.size, order, NoTrans, M, N, c["ldc"], c["offC"])
    assert same_bits(got[mask], bufs[2][mask])
    assert lib.device_fault() == 0


def test_beta_zero_does_not_upload_c_and_degenerate_cases(lib):
    M, N, K = 512, 600, 300
    A = torch.ones(M * K, dtype=torch.float64).pin_memory()
    B = torch.ones(K * N, dtype=torch.float64).pin_memory()
    C = torch.full((M * N,), float("nan"), dtype=torch.float64).pin_memory()
    k = (lib.clblasColumnMajor, lib.clblasNoTrans, lib.clblasNoTrans, M, N, K)
    assert lib.clblasB200DgemmHost(*k, 1.0, A, 0, M, B, 0, K, 0.0, C, 0, M) == lib.clblasSuccess
    torch.cuda.synchronize()
    assert torch.all(C == K)
    # alpha == 0: C <- beta*C, A and B are not touched (they may even be unreadable sizes)
    assert lib.clblasB200DgemmHost(*k, 0.0, A, 0, M, B, 0, K, 0.5, C, 0, M) == lib.clblasSuccess
    torch.cuda.synchronize()
    assert torch.all(C == K / 2)
    assert lib.clblasB200DgemmHost(*k, 1.0, None, 0, M, B, 0, K, 0.0, C, 0, M) == lib.clblasInvalidMatA
    assert lib.clblasB200DgemmHost(*k, 1.0, A, 0, M - 1, B, 0, K, 0.0, C, 0, M) == lib.clblasInvalidLeadDimA
    assert lib.clblasB200DgemmHost(*k, 1.0, A, 0, M, B, 0, K, 0.0, C, 0, M - 1) == lib.clblasInvalidLeadDimC
    assert lib.clblasB200DgemmHost(*k, 1.0, A, 0, M, B, 0, K, 0.0, C, 0, M, queues=[]) == lib.clblasInvalidCommandQueue


# --------------------------------------------------------------------------------- TRSM on host matrices
def run_trsm_host(cb, c, bufs):
    A, B = (torch.from_numpy(x).pin_memory() for x in bufs)
    fn = cb.clblasB200StrsmHost if c["prec"] == "s" else cb.clblasB200DtrsmHost
    st = fn(c["order"], c["side"], c["uplo"], c["transA"], c["diag"], c["M"], c["N"], c["alpha"], A, c["offA"], c["lda"],
            B, c["offB"], c["ldb"])
    torch.cuda.synchronize()
    return st, B.numpy().copy()


@pytest.mark.parametrize("prec", ["s", "d"])
def test_trsm_host_small_cases(lib, prec):
    """Every order / side / triangle / transposition / diagonal: same acceptance as the device routine (backward
    error within 4*M*u, NaN-poisoned triangle never read, padding of the host B untouched)."""
    for c in cases.sweep_trsm_cases(prec)[::4]:
        logical = cases.trsm_logical(c)
        bufs = cases.trsm_buffers(c, logical)
        st, got = run_trsm_host(lib, c, bufs)
        assert st == lib.clblasSuccess, (lib.STATUS_NAME.get(st, st), c)
        mask = oracle.outside_mask(got.size, c["order"], NoTrans, c["M"], c["N"], c["ldb"], c["offB"])
        assert same_bits(got[mask], bufs[1][mask]), c
        X = oracle.view(got, c["order"], NoTrans, c["M"], c["N"], c["ldb"], c["offB"])
        assert np.all(np.isfinite(X)), c
        T = cases.trsm_op_triangle(c, logical[0])
        assert oracle.trsm_backward_ratio(X, c["alpha"], T, logical[1], c["side"], cases.DT[prec]) <= 1.0, c


@pytest.mark.parametrize("side", [oracle.Left, oracle.Right])
def test_trsm_host_several_blocks(lib, side):
    """2048 x 9000 (Left) / 9000 x 2048 (Right): three blocks of right-hand sides through the pipeline."""
    M, N = (2048, 9000) if side == oracle.Left else (9000, 2048)
    c = cases.trsm_case("d", ColumnMajor, side, oracle.Lower, NoTrans, oracle.NonUnit, M, N, alpha=-2.0, pad=(3, 5), off=(2, 4), seed=91)
    logical = cases.trsm_logical(c)
    bufs = cases.trsm_buffers(c, logical)
    st, got = run_trsm_host(lib, c, bufs)
    assert st == lib.clblasSuccess
    mask = oracle.outside_mask(got.size, ColumnMajor, NoTrans, M, N, c["ldb"], c["offB"])
    assert same_bits(got[mask], bufs[1][mask])
    X = oracle.view(got, ColumnMajor, NoTrans, M, N, c["ldb"], c["offB"])
    T = cases.trsm_op_triangle(c, logical[0])
    assert oracle.trsm_backward_ratio(X, c["alpha"], T, logical[1], side, np.float64) <= 1.0
    assert lib.device_fault() == 0
