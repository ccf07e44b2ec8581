"""Complex TRSM parity on the GPU, through the C ABI, against the CPU oracle (the reference's
NaiveBlas::trsm on FloatComplex / DoubleComplex).

Inputs: diagonally dominant complex triangles with NaN outside the referenced triangle and on a unit
diagonal, so an illegal read poisons the result.  Acceptance: entrywise backward error
|alpha B - op(A) X| / (|op(A)||X| + |alpha||B|) <= 4*(2n)*u (n the order of A; a complex row sums 2n real
products per part), agreement with the oracle's solution within the forward bound that implies for these
well-conditioned systems, and padding / offset regions of B bit-untouched."""
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
    fn = cb.clblasCtrsm if c["prec"] == "c" else cb.clblasZtrsm
    st = fn(c["order"], c["side"], c["uplo"], c["transA"], c["diag"], c["M"], c["N"], c["alpha"], dA, c["offA"], c["lda"],
            dB, c["offB"], c["ldb"])
    torch.cuda.synchronize()
    return st, dB.cpu().numpy()


def check(cb, c, with_oracle=True):
    logical = cc.ctrsm_logical(c)
    bufs = cc.ctrsm_buffers(c, logical)
    st, got = run_gpu(cb, c, bufs)
    assert st == cb.clblasSuccess, (cb.STATUS_NAME.get(st, st), c)
    mask = oracle.outside_mask(got.size, c["order"], NoTrans, c["M"], c["N"], c["ldb"], c["offB"])
    assert same_bits(got[mask], bufs[1][mask]), c
    X = oracle.view(got, c["order"], NoTrans, c["M"], c["N"], c["ldb"], c["offB"])
    assert np.all(np.isfinite(X)), c
    T = cc.ctrsm_op_triangle(c, logical[0])
    ratio = cc.ctrsm_backward_ratio(c, X, T, logical[1])
    assert ratio <= 1.0, (ratio, c)
    if with_oracle:
        want = bufs[1].copy()
        oracle.ctrsm(c["order"], c["side"], c["uplo"], c["transA"], c["diag"], c["M"], c["N"], c["alpha"], bufs[0], c["offA"],
                     c["lda"], want, c["offB"], c["ldb"])
        Xo = oracle.view(want, c["order"], NoTrans, c["M"], c["N"], c["ldb"], c["offB"])
        scale = np.max(np.abs(Xo)) + 1e-30
        assert np.max(np.abs(X - Xo)) / scale <= 64 * 2 * T.shape[0] * oracle.unit_roundoff(cc.RDT[c["prec"]]), c
    return ratio


@pytest.mark.parametrize("prec", ["c", "z"])
def test_sweep_all_variants(lib, prec):
    """order x side x uplo x {N, T, C} x diag, sizes below / at / above the 64-row complex block."""
    for c in cc.sweep_ctrsm_cases(prec):
        check(lib, c)


@pytest.mark.parametrize("prec", ["c", "z"])
def test_large(lib, prec):
    """Several recursion levels on the TMA kernels; the oracle is skipped (O(n^2 N) on the CPU), the residual decides."""
    for c in (cc.ctrsm_case(prec, ColumnMajor, Left, Lower, NoTrans, NonUnit, 1024, 768, alpha=2 - 1j, seed=111),
              cc.ctrsm_case(prec, ColumnMajor, Left, Upper, ConjTrans, Unit, 1000, 600, alpha=1j, pad=(2, 4), off=(2, 4), seed=112),
              cc.ctrsm_case(prec, RowMajor, Right, Lower, Trans, NonUnit, 700, 1100, alpha=-1 + 0j, pad=(1, 3), off=(1, 3), seed=113),
              cc.ctrsm_case(prec, ColumnMajor, Right, Upper, ConjTrans, NonUnit, 900, 520, alpha=1 + 0j, seed=114)):
        check(lib, c, with_oracle=False)
    assert lib.device_fault() == 0


def test_status_codes_and_alpha_zero(lib):
    A = torch.eye(64, dtype=torch.complex128, device="cuda").reshape(-1).contiguous() * (2 + 0j)
    B = torch.full((64 * 8,), 4 + 2j, dtype=torch.complex128, device="cuda")
    k = (lib.clblasColumnMajor, lib.clblasLeft, lib.clblasLower, lib.clblasNoTrans, lib.clblasNonUnit, 64, 8)
    assert lib.clblasZtrsm(*k, 1 + 0j, None, 0, 64, B, 0, 64) == lib.clblasInvalidMatA
    assert lib.clblasZtrsm(*k, 1 + 0j, A, 0, 63, B, 0, 64) == lib.clblasInvalidLeadDimA
    assert lib.clblasZtrsm(*k, 1 + 0j, A, 0, 64, B, 0, 63) == lib.clblasInvalidLeadDimB
    assert lib.clblasZtrsm(*k, 1 + 0j, A, 0, 64, B, 0, 64, queues=[]) == lib.clblasInvalidCommandQueue
    assert lib.clblasZtrsm(*k, 1j, A, 0, 64, B, 0, 64) == lib.clblasSuccess
    torch.cuda.synchronize()
    assert torch.all(B == (-1 + 2j))          # (4 + 2i) * i / 2
    assert lib.clblasZtrsm(*k, 0j, A, 0, 64, B, 0, 64) == lib.clblasSuccess
    torch.cuda.synchronize()
    assert torch.all(B == 0)
