"""Complex GEMM parity on the GPU, through the C ABI, against the CPU oracle (the reference's
NaiveBlas::gemm on FloatComplex / DoubleComplex).

Integer-valued inputs (real and imaginary parts, alpha and beta too): every product and sum is exact,
so C must equal the oracle's.  Real-valued inputs: |C - C_exact| <= 4*(2K)*u*(|alpha||op(A)||op(B)| + |beta||C|)
entrywise (a complex product sums 2K real products per part).  Padding and offset regions hold NaN
and must keep their bits."""
import numpy as np
import pytest
import torch

import oracle
from oracle import ColumnMajor, ConjTrans, NoTrans, RowMajor, Trans
from tests import cases_complex as cc
from tests.gpu_util import dev, same_bits

pytestmark = pytest.mark.gpu


def run_gpu(cb, c, bufs):
    dA, dB, dC = (dev(x) for x in bufs)
    fn = cb.clblasCgemm if c["prec"] == "c" else cb.clblasZgemm
    st = fn(c["order"], c["transA"], c["transB"], c["M"], c["N"], c["K"], c["alpha"], dA, c["offA"], c["lda"],
            dB, c["offB"], c["ldb"], c["beta"], dC, c["offC"], c["ldc"])
    torch.cuda.synchronize()
    return st, dC.cpu().numpy()


def run_oracle(c, bufs):
    A, B, C = bufs
    C = C.copy()
    oracle.cgemm(c["order"], c["transA"], c["transB"], c["M"], c["N"], c["K"], c["alpha"], A, c["offA"], c["lda"],
                 B, c["offB"], c["ldb"], c["beta"], C, c["offC"], c["ldc"])
    return C


def outside_kept(c, before, after):
    mask = oracle.outside_mask(before.size, c["order"], NoTrans, c["M"], c["N"], c["ldc"], c["offC"])
    return same_bits(before[mask], after[mask])


@pytest.mark.parametrize("prec", ["c", "z"])
def test_sweep_exact_integer(lib, prec):
    for c in cc.sweep_cgemm_cases(prec, "int"):
        bufs = cc.cgemm_buffers(c)
        st, got = run_gpu(lib, c, bufs)
        assert st == lib.clblasSuccess, (lib.STATUS_NAME.get(st, st), c)
        assert np.array_equal(got, run_oracle(c, bufs), equal_nan=True), c
        assert outside_kept(c, bufs[2], got), c


@pytest.mark.parametrize("prec", ["c", "z"])
def test_sweep_real_valued(lib, prec):
    u = oracle.unit_roundoff(cc.RDT[prec])
    for c in cc.sweep_cgemm_cases(prec, "uniform")[::2]:
        logical = cc.cgemm_logical(c)
        bufs = cc.cgemm_buffers(c, logical)
        st, got = run_gpu(lib, c, bufs)
        assert st == lib.clblasSuccess
        assert outside_kept(c, bufs[2], got), c
        X = oracle.view(got, c["order"], NoTrans, c["M"], c["N"], c["ldc"], c["offC"]).astype(np.complex128)
        want, mag = cc.cgemm_exact(c, logical)
        assert np.all(np.abs(X - want) <= 4 * 2 * c["K"] * u * mag + 1e-300), c


@pytest.mark.parametrize("prec", ["c", "z"])
def test_large(lib, prec):
    """TMA kernels on the doubled real problem, all three operand treatments (in place, planar, expanded)."""
    for c in (cc.cgemm_case(prec, ColumnMajor, NoTrans, NoTrans, 1024, 768, 512, alpha=2 - 1j, beta=-1 + 0j, mode="int", seed=101),
              cc.cgemm_case(prec, ColumnMajor, ConjTrans, Trans, 1000, 900, 520, alpha=1 + 2j, beta=1j, pad=(2, 4, 6), off=(2, 4, 6),
                            mode="int", seed=102),
              cc.cgemm_case(prec, RowMajor, Trans, ConjTrans, 700, 1100, 300, alpha=-1j, beta=0j, pad=(1, 3, 1), off=(1, 1, 3),
                            mode="int", seed=103)):
        logical = cc.cgemm_logical(c)
        bufs = cc.cgemm_buffers(c, logical)
        st, got = run_gpu(lib, c, bufs)
        assert st == lib.clblasSuccess
        want, _ = cc.cgemm_exact(c, logical)
        X = oracle.view(got, c["order"], NoTrans, c["M"], c["N"], c["ldc"], c["offC"])
        assert np.array_equal(X.astype(np.complex128), want), c
        assert outside_kept(c, bufs[2], got), c
    assert lib.device_fault() == 0


def test_status_codes_and_degenerate(lib):
    A = torch.ones(64 * 16, dtype=torch.complex128, device="cuda")
    B = torch.ones(16 * 32, dtype=torch.complex128, device="cuda")
    C = torch.full((64 * 32,), 1 + 1j, dtype=torch.complex128, device="cuda")
    k = (lib.clblasColumnMajor, lib.clblasNoTrans, lib.clblasNoTrans, 64, 32, 16)
    assert lib.clblasZgemm(*k, 1j, None, 0, 64, B, 0, 16, 0j, C, 0, 64) == lib.clblasInvalidMatA
    assert lib.clblasZgemm(*k, 1j, A, 0, 63, B, 0, 16, 0j, C, 0, 64) == lib.clblasInvalidLeadDimA
    assert lib.clblasZgemm(*k, 1j, A, 0, 64, B, 0, 15, 0j, C, 0, 64) == lib.clblasInvalidLeadDimB
    assert lib.clblasZgemm(*k, 1j, A, 0, 64, B, 0, 16, 0j, C, 0, 63) == lib.clblasInvalidLeadDimC
    assert lib.clblasZgemm(*k, 1j, A, 0, 64, B, 0, 16, 0j, C, 0, 64, queues=[]) == lib.clblasInvalidCommandQueue
    # alpha == 0: C <- beta*C, A and B not referenced
    assert lib.clblasZgemm(*k, 0j, A, 0, 64, B, 0, 16, 2j, C, 0, 64) == lib.clblasSuccess
    torch.cuda.synchronize()
    assert torch.all(C == (-2 + 2j))
    assert lib.clblasZgemm(*k, 1j, A, 0, 64, B, 0, 16, 0j, C, 0, 64) == lib.clblasSuccess
    torch.cuda.synchronize()
    assert torch.all(C == 16j)
