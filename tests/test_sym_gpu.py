"""SYR2K and SYMM parity on the GPU, through the C ABI, against the CPU oracle.

Integer-valued inputs: every product and partial sum is exact, so the result must equal the oracle's
whatever the blocking.  Real-valued inputs: entrywise error within 4*k*u times the magnitude sum
(k = 2K for SYR2K, the order of A for SYMM).  NaN fills whatever must not be read or written: the
unreferenced triangle of C (SYR2K), of the symmetric A (SYMM), and all padding / offset regions."""
import numpy as np
import pytest
import torch

import oracle
from oracle import ColumnMajor, Left, Lower, NoTrans, Right, RowMajor, Trans, Upper
from tests import cases, cases_sym
from tests.gpu_util import dev, same_bits

pytestmark = pytest.mark.gpu


# ------------------------------------------------------------------------------------------- SYR2K
def syr2k_gpu(cb, c, bufs):
    dA, dB, dC = (dev(x) for x in bufs)
    fn = cb.clblasSsyr2k if c["prec"] == "s" else cb.clblasDsyr2k
    st = fn(c["order"], c["uplo"], c["trans"], c["N"], c["K"], c["alpha"], dA, c["offA"], c["lda"], dB, c["offB"], c["ldb"],
            c["beta"], dC, c["offC"], c["ldc"])
    torch.cuda.synchronize()
    return st, dC.cpu().numpy()


def syr2k_oracle(c, bufs):
    A, B, C = bufs
    C = C.copy()
    oracle.syr2k(c["order"], c["uplo"], c["trans"], c["N"], c["K"], c["alpha"], A, c["offA"], c["lda"], B, c["offB"], c["ldb"],
                 c["beta"], C, c["offC"], c["ldc"])
    return C


def tri_untouched(c, before, after):
    """Padding, offsets and the unreferenced triangle of the N x N matrix C kept their bits."""
    mask = oracle.outside_mask(before.size, c["order"], NoTrans, c["N"], c["N"], c["ldc"], c["offC"])
    if not same_bits(before[mask], after[mask]):
        return False
    b = oracle.view(before, c["order"], NoTrans, c["N"], c["N"], c["ldc"], c["offC"])
    a = oracle.view(after, c["order"], NoTrans, c["N"], c["N"], c["ldc"], c["offC"])
    other = cases_sym.other_triangle(c["N"], c["uplo"])
    return same_bits(np.ascontiguousarray(b[other]), np.ascontiguousarray(a[other]))


@pytest.mark.parametrize("prec", ["s", "d"])
def test_syr2k_sweep_exact_integer(lib, prec):
    for c in cases_sym.sweep_syr2k_cases(prec, "int"):
        bufs = cases_sym.syr2k_buffers(c)
        st, got = syr2k_gpu(lib, c, bufs)
        assert st == lib.clblasSuccess, (lib.STATUS_NAME.get(st, st), c)
        assert np.array_equal(got, syr2k_oracle(c, bufs), equal_nan=True), c
        assert tri_untouched(c, bufs[2], got), c


@pytest.mark.parametrize("prec", ["s", "d"])
def test_syr2k_sweep_real_valued(lib, prec):
    dt = cases.DT[prec]
    for c in cases_sym.sweep_syr2k_cases(prec, "uniform")[::2]:
        logical = cases_sym.syr2k_logical(c)
        bufs = cases_sym.syr2k_buffers(c, logical)
        st, got = syr2k_gpu(lib, c, bufs)
        assert st == lib.clblasSuccess
        assert tri_untouched(c, bufs[2], got), c
        opA, opB, C = (x.astype(np.float64) for x in logical)
        C = np.nan_to_num(C)
        X = oracle.view(got, c["order"], NoTrans, c["N"], c["N"], c["ldc"], c["offC"]).astype(np.float64)
        want = c["alpha"] * (opA @ opB.T + opB @ opA.T) + c["beta"] * C
        mag = abs(c["alpha"]) * (np.abs(opA) @ np.abs(opB).T + np.abs(opB) @ np.abs(opA).T) + abs(c["beta"]) * np.abs(C)
        tri = ~cases_sym.other_triangle(c["N"], c["uplo"])
        assert np.all(np.abs(X - want)[tri] <= (4 * 2 * c["K"] * oracle.unit_roundoff(dt) * mag)[tri] + 1e-300), c


@pytest.mark.parametrize("prec", ["s", "d"])
def test_syr2k_large(lib, prec):
    for c in (cases_sym.syr2k_case(prec, ColumnMajor, Upper, NoTrans, 2048, 600, alpha=2.0, beta=-1.0, mode="int", seed=91),
              cases_sym.syr2k_case(prec, RowMajor, Lower, Trans, 1900, 520, alpha=-1.0, beta=0.0, pad=(1, 2, 3), off=(2, 3, 5),
                                   mode="int", seed=92)):
        logical = cases_sym.syr2k_logical(c)
        bufs = cases_sym.syr2k_buffers(c, logical)
        st, got = syr2k_gpu(lib, c, bufs)
        assert st == lib.clblasSuccess
        opA, opB, C = (x.astype(np.float64) for x in logical)
        want = c["alpha"] * (opA @ opB.T + opB @ opA.T) + c["beta"] * np.nan_to_num(C)
        X = oracle.view(got, c["order"], NoTrans, c["N"], c["N"], c["ldc"], c["offC"])
        tri = ~cases_sym.other_triangle(c["N"], c["uplo"])
        assert np.array_equal(X[tri].astype(np.float64), want[tri]), c
        assert tri_untouched(c, bufs[2], got), c
    assert lib.device_fault() == 0


# -------------------------------------------------------------------------------------------- SYMM
def symm_gpu(cb, c, bufs):
    dA, dB, dC = (dev(x) for x in bufs)
    fn = cb.clblasSsymm if c["prec"] == "s" else cb.clblasDsymm
    st = fn(c["order"], c["side"], c["uplo"], c["M"], c["N"], c["alpha"], dA, c["offA"], c["lda"], dB, c["offB"], c["ldb"],
            c["beta"], dC, c["offC"], c["ldc"])
    torch.cuda.synchronize()
    return st, dC.cpu().numpy()


def symm_oracle(c, bufs):
    A, B, C = bufs
    C = C.copy()
    oracle.symm(c["order"], c["side"], c["uplo"], c["M"], c["N"], c["alpha"], A, c["offA"], c["lda"], B, c["offB"], c["ldb"],
                c["beta"], C, c["offC"], c["ldc"])
    return C


@pytest.mark.parametrize("prec", ["s", "d"])
def test_symm_sweep_exact_integer(lib, prec):
    for c in cases_sym.sweep_symm_cases(prec, "int"):
        bufs = cases_sym.symm_buffers(c)
        st, got = symm_gpu(lib, c, bufs)
        assert st == lib.clblasSuccess, (lib.STATUS_NAME.get(st, st), c)
        assert np.array_equal(got, symm_oracle(c, bufs), equal_nan=True), c
        mask = oracle.outside_mask(got.size, c["order"], NoTrans, c["M"], c["N"], c["ldc"], c["offC"])
        assert same_bits(got[mask], bufs[2][mask]), c


@pytest.mark.parametrize("prec", ["s", "d"])
def test_symm_sweep_real_valued(lib, prec):
    dt = cases.DT[prec]
    for c in cases_sym.sweep_symm_cases(prec, "uniform")[::2]:
        logical = cases_sym.symm_logical(c)
        bufs = cases_sym.symm_buffers(c, logical)
        st, got = symm_gpu(lib, c, bufs)
        assert st == lib.clblasSuccess
        mask = oracle.outside_mask(got.size, c["order"], NoTrans, c["M"], c["N"], c["ldc"], c["offC"])
        assert same_bits(got[mask], bufs[2][mask]), c
        X = oracle.view(got, c["order"], NoTrans, c["M"], c["N"], c["ldc"], c["offC"]).astype(np.float64)
        want, mag = cases_sym.symm_exact(c, logical)
        n = c["M"] if c["side"] == Left else c["N"]
        assert np.all(np.abs(X - want) <= 4 * n * oracle.unit_roundoff(dt) * mag + 1e-300), c


@pytest.mark.parametrize("prec", ["s", "d"])
def test_symm_large(lib, prec):
    for c in (cases_sym.symm_case(prec, ColumnMajor, Left, Lower, 2048, 1024, alpha=2.0, beta=-1.0, mode="int", seed=93),
              cases_sym.symm_case(prec, RowMajor, Right, Upper, 1000, 1500, alpha=-1.0, beta=0.0, pad=(1, 2, 3), off=(2, 3, 5),
                                  mode="int", seed=94)):
        logical = cases_sym.symm_logical(c)
        st, got = symm_gpu(lib, c, cases_sym.symm_buffers(c, logical))
        assert st == lib.clblasSuccess
        want, _ = cases_sym.symm_exact(c, logical)
        X = oracle.view(got, c["order"], NoTrans, c["M"], c["N"], c["ldc"], c["offC"])
        assert np.array_equal(X.astype(np.float64), want), c
    assert lib.device_fault() == 0


def test_status_codes(lib):
    A = torch.ones(64 * 64, dtype=torch.float64, device="cuda")
    B = torch.ones(64 * 16, dtype=torch.float64, device="cuda")
    C = torch.zeros(64 * 64, dtype=torch.float64, device="cuda")
    k = (lib.clblasColumnMajor, lib.clblasLower, lib.clblasNoTrans, 64, 16, 1.0)
    assert lib.clblasDsyr2k(*k, None, 0, 64, B, 0, 64, 0.0, C, 0, 64) == lib.clblasInvalidMatA
    assert lib.clblasDsyr2k(*k, B, 0, 64, None, 0, 64, 0.0, C, 0, 64) == lib.clblasInvalidMatB
    assert lib.clblasDsyr2k(*k, B, 0, 64, B, 0, 63, 0.0, C, 0, 64) == lib.clblasInvalidLeadDimB
    assert lib.clblasDsyr2k(*k, B, 0, 64, B, 0, 64, 0.0, C, 0, 63) == lib.clblasInvalidLeadDimC
    assert lib.clblasDsyr2k(*k, B, 0, 64, B, 0, 64, 0.0, C, 0, 64) == lib.clblasSuccess
    torch.cuda.synchronize()
    c = C.reshape(64, 64).T
    assert torch.all(torch.tril(c) == 32.0 * torch.tril(torch.ones_like(c))) and torch.all(torch.triu(c, 1) == 0.0)
    m = (lib.clblasColumnMajor, lib.clblasLeft, lib.clblasUpper, 64, 16, 1.0)
    D = torch.zeros(64 * 16, dtype=torch.float64, device="cuda")
    assert lib.clblasDsymm(*m, None, 0, 64, B, 0, 64, 0.0, D, 0, 64) == lib.clblasInvalidMatA
    assert lib.clblasDsymm(*m, A, 0, 63, B, 0, 64, 0.0, D, 0, 64) == lib.clblasInvalidLeadDimA
    assert lib.clblasDsymm(*m, A, 0, 64, B, 0, 64, 0.0, None, 0, 64) == lib.clblasInvalidMatC
    assert lib.clblasDsymm(*m, A, 0, 64, B, 0, 64, 0.0, D, 0, 64) == lib.clblasSuccess
    torch.cuda.synchronize()
    assert torch.all(D == 64.0)
