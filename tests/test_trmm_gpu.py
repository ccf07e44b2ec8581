"""TRMM parity on the GPU, through the C ABI, against the CPU oracle (the reference's NaiveBlas::trmm).

Integer-valued inputs: every product and partial sum is exact, so the result must equal the oracle's
bit for bit whatever the blocking.  Real-valued inputs: entrywise |X - X_exact| <= 4*n*u*(|alpha||op(A)||B|),
n the order of the triangle.  A holds NaN outside the referenced triangle and on a unit diagonal; the
padding / offset regions of B are NaN and must keep their bits."""
import numpy as np
import pytest
import torch

import oracle
from oracle import ColumnMajor, Left, Lower, NonUnit, NoTrans, Right, RowMajor, Trans, Unit, Upper
from tests import cases, cases_trmm
from tests.gpu_util import dev, same_bits

pytestmark = pytest.mark.gpu


def run_gpu(cb, c, bufs):
    A, B = bufs
    dA, dB = dev(A), dev(B)
    fn = cb.clblasStrmm if c["prec"] == "s" else cb.clblasDtrmm
    st = fn(c["order"], c["side"], c["uplo"], c["transA"], c["diag"], c["M"], c["N"], c["alpha"], dA, c["offA"], c["lda"],
            dB, c["offB"], c["ldb"])
    torch.cuda.synchronize()
    return st, dB.cpu().numpy()


def run_oracle(c, bufs):
    A, B = bufs
    B = B.copy()
    oracle.trmm(c["order"], c["side"], c["uplo"], c["transA"], c["diag"], c["M"], c["N"], c["alpha"], A, c["offA"], c["lda"],
                B, c["offB"], c["ldb"])
    return B


@pytest.mark.parametrize("prec", ["s", "d"])
def test_sweep_exact_integer(lib, prec):
    for c in cases_trmm.sweep_trmm_cases(prec, "int"):
        bufs = cases_trmm.trmm_buffers(c)
        st, got = run_gpu(lib, c, bufs)
        assert st == lib.clblasSuccess, (lib.STATUS_NAME.get(st, st), c)
        # equal values everywhere (an exact zero may carry either sign: the blocked evaluation adds a
        # partial product to a partial product where the oracle scales one running sum), and
        # bit-identical outside the matrix
        assert np.array_equal(got, run_oracle(c, bufs), equal_nan=True), c
        mask = oracle.outside_mask(got.size, c["order"], NoTrans, c["M"], c["N"], c["ldb"], c["offB"])
        assert same_bits(got[mask], bufs[1][mask]), c


@pytest.mark.parametrize("prec", ["s", "d"])
def test_sweep_real_valued(lib, prec):
    dt = cases.DT[prec]
    for c in cases_trmm.sweep_trmm_cases(prec, "uniform")[::3]:
        logical = cases_trmm.trmm_logical(c)
        bufs = cases_trmm.trmm_buffers(c, logical)
        st, got = run_gpu(lib, c, bufs)
        assert st == lib.clblasSuccess
        mask = oracle.outside_mask(got.size, c["order"], NoTrans, c["M"], c["N"], c["ldb"], c["offB"])
        assert np.array_equal(bufs[1][mask].view(np.uint8), got[mask].view(np.uint8)), c
        X = oracle.view(got, c["order"], NoTrans, c["M"], c["N"], c["ldb"], c["offB"]).astype(np.float64)
        A, B = logical
        want, T = cases_trmm.trmm_exact(c, A, B)
        mag = abs(c["alpha"]) * (np.abs(T) @ np.abs(B.astype(np.float64)) if c["side"] == Left else np.abs(B.astype(np.float64)) @ np.abs(T))
        n = T.shape[0]
        assert np.all(np.abs(X - want) <= 4 * n * oracle.unit_roundoff(dt) * mag + 1e-300), c


@pytest.mark.parametrize("prec", ["s", "d"])
def test_large_left_lower(lib, prec):
    """Order 2048 with 1024 columns: several recursion levels, TMA kernels, in-place leaves."""
    c = cases_trmm.trmm_case(prec, ColumnMajor, Left, Lower, NoTrans, NonUnit, 2048, 1024, alpha=2.0, mode="int", seed=71)
    logical = cases_trmm.trmm_logical(c)
    st, got = run_gpu(lib, c, cases_trmm.trmm_buffers(c, logical))
    assert st == lib.clblasSuccess
    want, _ = cases_trmm.trmm_exact(c, *logical)
    assert np.array_equal(oracle.view(got, ColumnMajor, NoTrans, 2048, 1024, c["ldb"], 0), want.astype(cases.DT[prec]))
    c = cases_trmm.trmm_case(prec, RowMajor, Right, Upper, Trans, Unit, 1000, 1500, alpha=-1.0, pad=(1, 3), off=(2, 5), mode="int", seed=72)
    logical = cases_trmm.trmm_logical(c)
    st, got = run_gpu(lib, c, cases_trmm.trmm_buffers(c, logical))
    assert st == lib.clblasSuccess
    want, _ = cases_trmm.trmm_exact(c, *logical)
    assert np.array_equal(oracle.view(got, RowMajor, NoTrans, 1000, 1500, c["ldb"], c["offB"]), want.astype(cases.DT[prec]))
    assert lib.device_fault() == 0


def test_status_codes(lib):
    A = torch.eye(64, dtype=torch.float64, device="cuda").reshape(-1).contiguous()
    B = torch.ones(64 * 8, dtype=torch.float64, device="cuda")
    args = (lib.clblasColumnMajor, lib.clblasLeft, lib.clblasLower, lib.clblasNoTrans, lib.clblasNonUnit, 64, 8, 2.0)
    assert lib.clblasDtrmm(*args, None, 0, 64, B, 0, 64) == lib.clblasInvalidMatA
    assert lib.clblasDtrmm(*args, A, 0, 64, None, 0, 64) == lib.clblasInvalidMatB
    assert lib.clblasDtrmm(*args, A, 0, 63, B, 0, 64) == lib.clblasInvalidLeadDimA
    assert lib.clblasDtrmm(*args, A, 0, 64, B, 0, 63) == lib.clblasInvalidLeadDimB
    assert lib.clblasDtrmm(*args, A, 0, 64, B, 0, 64) == lib.clblasSuccess
    torch.cuda.synchronize()
    assert torch.all(B == 2.0)
