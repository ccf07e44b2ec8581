"""Complex SYRK / HERK / SYR2K / HER2K / SYMM / HEMM parity on the GPU, through the C ABI, against the CPU oracle.

Integer-valued inputs: every product and sum is exact, so the referenced triangle (the whole matrix for SYMM / HEMM)
must equal the oracle's.  Real-valued inputs: entrywise error within 4*k*u times the magnitude sum, k the number of real
products per part.  NaN fills whatever must not be read or written: the other triangle of C (rank-k updates) or of A
(SYMM / HEMM) and all padding; HEMM's A also carries garbage imaginary parts on its diagonal, which must be ignored;
Hermitian results must have an exactly real diagonal."""
import numpy as np
import pytest
import torch

import oracle
from oracle import ColumnMajor, ConjTrans, Left, Lower, NoTrans, Right, RowMajor, Trans, Upper
from tests import cases_complex as cc
from tests.gpu_util import dev, same_bits

pytestmark = pytest.mark.gpu


def run_rank_gpu(cb, c, bufs):
    dA, dB, dC = (dev(x) for x in bufs)
    fn = getattr(cb, f"clblas{c['prec'].upper()}{c['kind']}")
    if c["kind"] in ("syrk", "herk"):
        st = fn(c["order"], c["uplo"], c["trans"], c["N"], c["K"], c["alpha"], dA, c["offA"], c["lda"], c["beta"], dC, c["offC"], c["ldc"])
    else:
        st = fn(c["order"], c["uplo"], c["trans"], c["N"], c["K"], c["alpha"], dA, c["offA"], c["lda"], dB, c["offB"], c["ldb"],
                c["beta"], dC, c["offC"], c["ldc"])
    torch.cuda.synchronize()
    return st, dC.cpu().numpy()


def run_rank_oracle(c, bufs):
    A, B, C = bufs
    C = C.copy()
    herm = c["kind"] in ("herk", "her2k")
    if c["kind"] in ("syrk", "herk"):
        oracle.csyrk(c["order"], c["uplo"], c["trans"], c["N"], c["K"], c["alpha"], A, c["offA"], c["lda"], c["beta"], C, c["offC"],
                     c["ldc"], herm=herm)
    else:
        oracle.csyr2k(c["order"], c["uplo"], c["trans"], c["N"], c["K"], c["alpha"], A, c["offA"], c["lda"], B, c["offB"], c["ldb"],
                      c["beta"], C, c["offC"], c["ldc"], herm=herm)
    return C


def untouched(c, before, after):
    n = c["N"]
    mask = oracle.outside_mask(before.size, c["order"], NoTrans, n, n, c["ldc"], c["offC"])
    if not same_bits(before[mask], after[mask]):
        return False
    b = oracle.view(before, c["order"], NoTrans, n, n, c["ldc"], c["offC"])
    a = oracle.view(after, c["order"], NoTrans, n, n, c["ldc"], c["offC"])
    other = cc._other_triangle(n, c["uplo"])
    return same_bits(np.ascontiguousarray(b[other]), np.ascontiguousarray(a[other]))


@pytest.mark.parametrize("kind", ["syrk", "herk", "syr2k", "her2k"])
@pytest.mark.parametrize("prec", ["c", "z"])
def test_rank_updates_exact_integer(lib, kind, prec):
    for c in cc.sweep_crank_cases(kind, prec, "int"):
        bufs = cc.crank_buffers(c)
        st, got = run_rank_gpu(lib, c, bufs)
        assert st == lib.clblasSuccess, (lib.STATUS_NAME.get(st, st), c)
        assert np.array_equal(got, run_rank_oracle(c, bufs), equal_nan=True), c
        assert untouched(c, bufs[2], got), c


@pytest.mark.parametrize("kind", ["syrk", "herk", "syr2k", "her2k"])
@pytest.mark.parametrize("prec", ["c", "z"])
def test_rank_updates_real_valued(lib, kind, prec):
    u = oracle.unit_roundoff(cc.RDT[prec])
    for c in cc.sweep_crank_cases(kind, prec, "uniform")[::2]:
        logical = cc.crank_logical(c)
        bufs = cc.crank_buffers(c, logical)
        st, got = run_rank_gpu(lib, c, bufs)
        assert st == lib.clblasSuccess
        assert untouched(c, bufs[2], got), c
        X = oracle.view(got, c["order"], NoTrans, c["N"], c["N"], c["ldc"], c["offC"]).astype(np.complex128)
        want, mag = cc.crank_exact(c, logical)
        tri = ~cc._other_triangle(c["N"], c["uplo"])
        k = c["K"] * (4 if kind in ("syr2k", "her2k") else 2)
        assert np.all(np.abs(X - want)[tri] <= (4 * k * u * mag)[tri] + 1e-300), c
        if kind in ("herk", "her2k"):
            assert np.all(X.diagonal().imag == 0.0), c


@pytest.mark.parametrize("prec", ["c", "z"])
def test_rank_updates_large(lib, prec):
    for c in (cc.crank_case("syrk", prec, ColumnMajor, Lower, NoTrans, 1024, 520, 2 - 1j, -1 + 0j, mode="int", seed=121),
              cc.crank_case("herk", prec, RowMajor, Upper, ConjTrans, 900, 700, -1.0, 2.0, pad=(1, 0, 3), off=(2, 0, 5), mode="int", seed=122),
              cc.crank_case("syr2k", prec, ColumnMajor, Upper, Trans, 1000, 300, 1j, 0j, pad=(2, 4, 6), off=(2, 4, 6), mode="int", seed=123),
              cc.crank_case("her2k", prec, RowMajor, Lower, NoTrans, 700, 520, 1 + 2j, -1.0, pad=(1, 3, 1), off=(1, 1, 3), mode="int", seed=124)):
        logical = cc.crank_logical(c)
        bufs = cc.crank_buffers(c, logical)
        st, got = run_rank_gpu(lib, c, bufs)
        assert st == lib.clblasSuccess
        want, _ = cc.crank_exact(c, logical)
        X = oracle.view(got, c["order"], NoTrans, c["N"], c["N"], c["ldc"], c["offC"])
        tri = ~cc._other_triangle(c["N"], c["uplo"])
        assert np.array_equal(X[tri].astype(np.complex128), want[tri]), c
        assert untouched(c, bufs[2], got), c
    assert lib.device_fault() == 0


def run_symm_gpu(cb, c, bufs):
    dA, dB, dC = (dev(x) for x in bufs)
    fn = getattr(cb, f"clblas{c['prec'].upper()}{c['kind']}")
    st = fn(c["order"], c["side"], c["uplo"], c["M"], c["N"], c["alpha"], dA, c["offA"], c["lda"], dB, c["offB"], c["ldb"],
            c["beta"], dC, c["offC"], c["ldc"])
    torch.cuda.synchronize()
    return st, dC.cpu().numpy()


@pytest.mark.parametrize("kind", ["symm", "hemm"])
@pytest.mark.parametrize("prec", ["c", "z"])
def test_symm_hemm(lib, kind, prec):
    u = oracle.unit_roundoff(cc.RDT[prec])
    for mode in ("int", "uniform"):
        for c in cc.sweep_csymm_cases(kind, prec, mode)[:: (1 if mode == "int" else 2)]:
            logical = cc.csymm_logical(c)
            bufs = cc.csymm_buffers(c, logical)
            st, got = run_symm_gpu(lib, c, bufs)
            assert st == lib.clblasSuccess, (lib.STATUS_NAME.get(st, st), c)
            mask = oracle.outside_mask(got.size, c["order"], NoTrans, c["M"], c["N"], c["ldc"], c["offC"])
            assert same_bits(got[mask], bufs[2][mask]), c
            X = oracle.view(got, c["order"], NoTrans, c["M"], c["N"], c["ldc"], c["offC"]).astype(np.complex128)
            want, mag = cc.csymm_exact(c, logical)
            if mode == "int":
                assert np.array_equal(X, want), c
            else:
                n = c["M"] if c["side"] == Left else c["N"]
                assert np.all(np.abs(X - want) <= 4 * 2 * n * u * mag + 1e-300), c


def test_status_codes(lib):
    A = torch.ones(64 * 16, dtype=torch.complex128, device="cuda")
    C = torch.zeros(64 * 64, dtype=torch.complex128, device="cuda")
    k = (lib.clblasColumnMajor, lib.clblasLower)
    # a symmetric update refuses ConjTrans, a Hermitian one Trans
    assert lib.clblasZsyrk(*k, lib.clblasConjTrans, 64, 16, 1 + 0j, A, 0, 64, 0j, C, 0, 64) == lib.clblasInvalidValue
    assert lib.clblasZherk(*k, lib.clblasTrans, 64, 16, 1.0, A, 0, 64, 0.0, C, 0, 64) == lib.clblasInvalidValue
    assert lib.clblasZher2k(*k, lib.clblasTrans, 64, 16, 1 + 0j, A, 0, 64, A, 0, 64, 0.0, C, 0, 64) == lib.clblasInvalidValue
    assert lib.clblasZsyrk(*k, lib.clblasNoTrans, 64, 16, 1 + 0j, None, 0, 64, 0j, C, 0, 64) == lib.clblasInvalidMatA
    assert lib.clblasZsyrk(*k, lib.clblasNoTrans, 64, 16, 1 + 0j, A, 0, 63, 0j, C, 0, 64) == lib.clblasInvalidLeadDimA
    assert lib.clblasZherk(*k, lib.clblasNoTrans, 64, 16, 2.0, A, 0, 64, 0.0, C, 0, 64) == lib.clblasSuccess
    torch.cuda.synchronize()
    c = C.reshape(64, 64).T
    assert torch.all(torch.tril(c) == 32.0 * torch.tril(torch.ones_like(c))) and torch.all(torch.triu(c, 1) == 0)
