"""Complex TRMM parity on the GPU, through the C ABI, against the CPU oracle (the reference's NaiveBlas::trmm on
FloatComplex / DoubleComplex).  Integer inputs: equal to the oracle whatever the blocking; real inputs: entrywise
|X - X_exact| <= 4*(2n)*u*|alpha||op(A)||B|.  A holds NaN outside the referenced triangle and on a unit diagonal;
padding / offset regions of B are NaN and keep their bits."""
import numpy as np
import pytest
import torch

import oracle
from oracle import ColumnMajor, ConjTrans, Left, Lower, NonUnit, NoTrans, Right, RowMajor, Trans, Unit, Upper
from tests import cases_complex as cc
from tests.gpu_util import dev, same_bits

pytestmark = pytest.mark.gpu


def run_gpu(cb, c, bufs):
    dA, dB = (dev(x) for x in bufs)
    fn = cb.clblasCtrmm if c["prec"] == "c" else cb.clblasZtrmm
    st = fn(c["order"], c["side"], c["uplo"], c["transA"], c["diag"], c["M"], c["N"], c["alpha"], dA, c["offA"], c["lda"],
            dB, c["offB"], c["ldb"])
    torch.cuda.synchronize()
    return st, dB.cpu().numpy()


@pytest.mark.parametrize("prec", ["c", "z"])
def test_sweep_exact_integer(lib, prec):
    for c in cc.sweep_ctrmm_cases(prec, "int"):
        bufs = cc.ctrmm_buffers(c)
        st, got = run_gpu(lib, c, bufs)
        assert st == lib.clblasSuccess, (lib.STATUS_NAME.get(st, st), c)
        want = bufs[1].copy()
        oracle.ctrmm(c["order"], c["side"], c["uplo"], c["transA"], c["diag"], c["M"], c["N"], c["alpha"], bufs[0], c["offA"],
                     c["lda"], want, c["offB"], c["ldb"])
        assert np.array_equal(got, want, equal_nan=True), c
        mask = oracle.outside_mask(got.size, c["order"], NoTrans, c["M"], c["N"], c["ldb"], c["offB"])
        assert same_bits(got[mask], bufs[1][mask]), c


@pytest.mark.parametrize("prec", ["c", "z"])
def test_sweep_real_valued(lib, prec):
    u = oracle.unit_roundoff(cc.RDT[prec])
    for c in cc.sweep_ctrmm_cases(prec, "uniform")[::3]:
        logical = cc.ctrmm_logical(c)
        bufs = cc.ctrmm_buffers(c, logical)
        st, got = run_gpu(lib, c, bufs)
        assert st == lib.clblasSuccess
        X = oracle.view(got, c["order"], NoTrans, c["M"], c["N"], c["ldb"], c["offB"]).astype(np.complex128)
        want, mag, T = cc.ctrmm_exact(c, logical)
        assert np.all(np.abs(X - want) <= 4 * 2 * T.shape[0] * u * mag + 1e-300), c


@pytest.mark.parametrize("prec", ["c", "z"])
def test_large(lib, prec):
    for c in (cc.ctrmm_case(prec, ColumnMajor, Left, Lower, NoTrans, NonUnit, 1024, 768, alpha=2 - 1j, mode="int", seed=131),
              cc.ctrmm_case(prec, ColumnMajor, Left, Upper, ConjTrans, Unit, 1000, 600, alpha=1j, pad=(2, 4), off=(2, 4), mode="int", seed=132),
              cc.ctrmm_case(prec, RowMajor, Right, Lower, Trans, NonUnit, 700, 1100, alpha=-1 + 0j, pad=(1, 3), off=(1, 3), mode="int", seed=133)):
        logical = cc.ctrmm_logical(c)
        st, got = run_gpu(lib, c, cc.ctrmm_buffers(c, logical))
        assert st == lib.clblasSuccess
        want, _, _ = cc.ctrmm_exact(c, logical)
        X = oracle.view(got, c["order"], NoTrans, c["M"], c["N"], c["ldb"], c["offB"])
        assert np.array_equal(X.astype(np.complex128), want), c
    assert lib.device_fault() == 0
