"""SYRK parity on the GPU, through the C ABI, against the CPU oracle (the reference's NaiveBlas::syrk).

Integer-valued inputs: every product and partial sum is exact, so the referenced triangle must equal
the oracle's whatever the blocking.  Real-valued inputs: entrywise
|C - C_exact| <= 4*K*u*(|alpha||op(A)||op(A)|^T + |beta||C|).  The triangle of C that SYRK does not
reference holds NaN, the padding / offset regions too; all of them must keep their bits."""
import numpy as np
import pytest
import torch

import oracle
from oracle import ColumnMajor, Lower, NoTrans, RowMajor, Trans, Upper
from tests import cases, cases_syrk
from tests.gpu_util import dev, same_bits

pytestmark = pytest.mark.gpu


def run_gpu(cb, c, bufs):
    A, C = bufs
    dA, dC = dev(A), dev(C)
    fn = cb.clblasSsyrk if c["prec"] == "s" else cb.clblasDsyrk
    st = fn(c["order"], c["uplo"], c["trans"], c["N"], c["K"], c["alpha"], dA, c["offA"], c["lda"], c["beta"], dC, c["offC"],
            c["ldc"])
    torch.cuda.synchronize()
    return st, dC.cpu().numpy()


def run_oracle(c, bufs):
    A, C = bufs
    C = C.copy()
    oracle.syrk(c["order"], c["uplo"], c["trans"], c["N"], c["K"], c["alpha"], A, c["offA"], c["lda"], c["beta"], C,
                c["offC"], c["ldc"])
    return C


def tri_mask(c):
    N = c["N"]
    return np.tril(np.ones((N, N), dtype=bool)) if c["uplo"] == Lower else np.triu(np.ones((N, N), dtype=bool))


def untouched(c, before, after):
    """Padding, offsets and the unreferenced triangle kept their bits."""
    mask = oracle.outside_mask(before.size, c["order"], NoTrans, c["N"], c["N"], c["ldc"], c["offC"])
    if not same_bits(before[mask], after[mask]):
        return False
    b = oracle.view(before, c["order"], NoTrans, c["N"], c["N"], c["ldc"], c["offC"])
    a = oracle.view(after, c["order"], NoTrans, c["N"], c["N"], c["ldc"], c["offC"])
    other = ~tri_mask(c)
    return same_bits(np.ascontiguousarray(b[other]), np.ascontiguousarray(a[other]))


@pytest.mark.parametrize("prec", ["s", "d"])
def test_sweep_exact_integer(lib, prec):
    for c in cases_syrk.sweep_syrk_cases(prec, "int"):
        bufs = cases_syrk.syrk_buffers(c)
        st, got = run_gpu(lib, c, bufs)
        assert st == lib.clblasSuccess, (lib.STATUS_NAME.get(st, st), c)
        assert np.array_equal(got, run_oracle(c, bufs), equal_nan=True), c
        assert untouched(c, bufs[1], got), c


@pytest.mark.parametrize("prec", ["s", "d"])
def test_sweep_real_valued(lib, prec):
    dt = cases.DT[prec]
    for c in cases_syrk.sweep_syrk_cases(prec, "uniform")[::2]:
        logical = cases_syrk.syrk_logical(c)
        bufs = cases_syrk.syrk_buffers(c, logical)
        st, got = run_gpu(lib, c, bufs)
        assert st == lib.clblasSuccess
        assert untouched(c, bufs[1], got), c
        opA, C = (x.astype(np.float64) for x in logical)
        X = oracle.view(got, c["order"], NoTrans, c["N"], c["N"], c["ldc"], c["offC"]).astype(np.float64)
        want = c["alpha"] * (opA @ opA.T) + c["beta"] * np.nan_to_num(C)
        mag = abs(c["alpha"]) * (np.abs(opA) @ np.abs(opA).T) + abs(c["beta"]) * np.abs(np.nan_to_num(C))
        tri = tri_mask(c)
        assert np.all(np.abs(X - want)[tri] <= (4 * c["K"] * oracle.unit_roundoff(dt) * mag)[tri] + 1e-300), c


@pytest.mark.parametrize("prec", ["s", "d"])
def test_large(lib, prec):
    """Order 2048 / 1900: several recursion levels, TMA kernels on the off-diagonal blocks, merged leaves."""
    for c in (cases_syrk.syrk_case(prec, ColumnMajor, Lower, NoTrans, 2048, 1024, alpha=2.0, beta=-1.0, mode="int", seed=81),
              cases_syrk.syrk_case(prec, RowMajor, Upper, Trans, 1900, 700, alpha=-1.0, beta=0.0, pad=(1, 3), off=(2, 5),
                                   mode="int", seed=82)):
        logical = cases_syrk.syrk_logical(c)
        bufs = cases_syrk.syrk_buffers(c, logical)
        st, got = run_gpu(lib, c, bufs)
        assert st == lib.clblasSuccess
        opA, C = (x.astype(np.float64) for x in logical)
        want = c["alpha"] * (opA @ opA.T) + c["beta"] * np.nan_to_num(C)
        X = oracle.view(got, c["order"], NoTrans, c["N"], c["N"], c["ldc"], c["offC"])
        tri = tri_mask(c)
        assert np.array_equal(X[tri].astype(np.float64), want[tri]), c
        assert untouched(c, bufs[1], got), c
    assert lib.device_fault() == 0


def test_alpha_zero_scales_triangle_only(lib):
    c = cases_syrk.syrk_case("d", ColumnMajor, Upper, NoTrans, 300, 40, alpha=0.0, beta=3.0, pad=(0, 2), mode="int", seed=83)
    bufs = cases_syrk.syrk_buffers(c)
    st, got = run_gpu(lib, c, bufs)
    assert st == lib.clblasSuccess
    assert np.array_equal(got, run_oracle(c, bufs), equal_nan=True)
    assert untouched(c, bufs[1], got)


def test_status_codes(lib):
    A = torch.ones(64 * 16, dtype=torch.float64, device="cuda")
    C = torch.zeros(64 * 64, dtype=torch.float64, device="cuda")
    args = (lib.clblasColumnMajor, lib.clblasLower, lib.clblasNoTrans, 64, 16, 1.0)
    assert lib.clblasDsyrk(*args, None, 0, 64, 0.0, C, 0, 64) == lib.clblasInvalidMatA
    assert lib.clblasDsyrk(*args, A, 0, 64, 0.0, None, 0, 64) == lib.clblasInvalidMatC
    assert lib.clblasDsyrk(*args, A, 0, 63, 0.0, C, 0, 64) == lib.clblasInvalidLeadDimA
    assert lib.clblasDsyrk(*args, A, 0, 64, 0.0, C, 0, 63) == lib.clblasInvalidLeadDimC
    assert lib.clblasDsyrk(*args, A, 0, 64, 0.0, C, 1 << 30, 64) == lib.clblasInsufficientMemMatC
    assert lib.clblasDsyrk(*args, A, 0, 64, 0.0, C, 0, 64) == lib.clblasSuccess
    torch.cuda.synchronize()
    c = C.reshape(64, 64).T  # column-major view
    assert torch.all(torch.tril(c) == 16.0 * torch.tril(torch.ones_like(c)))
    assert torch.all(torch.triu(c, 1) == 0.0)
