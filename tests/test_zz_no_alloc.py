"""clblasB200DtrsmNoAlloc -- the DTRSM entry point for callers that cannot allocate device memory
while they run (all GPU memory already owned by their own pool, or a fixed memory budget).  It
must give what clblasDtrsm gives, call after call, although every call reuses one resident
scratch array; and it must refuse, cleanly, problems larger than that array.

Collected last on purpose: a failure here cannot hide the result of any other test."""
import numpy as np
import pytest

import oracle
from oracle import ColumnMajor, Left, Lower, NonUnit, NoTrans, Right, RowMajor, Trans, Unit, Upper
from tests import cases
from tests.gpu_util import dev, outside_untouched, run_trsm_gpu

pytestmark = pytest.mark.gpu


def _run_noalloc(cb, c, bufs):
    import torch
    A, B = bufs
    dA, dB = dev(A), dev(B)
    st = cb.clblasB200DtrsmNoAlloc(c["order"], c["side"], c["uplo"], c["transA"], c["diag"], c["M"], c["N"], c["alpha"],
                                   dA, c["offA"], c["lda"], dB, c["offB"], c["ldb"])
    torch.cuda.synchronize()
    return st, dB.cpu().numpy()


def test_matches_allocating_entry_point_on_consecutive_calls(lib):
    """Two calls in a row (different shapes, so the second finds the first one's data in the scratch
    array), each compared with clblasDtrsm on the same inputs and with the backward-error bound."""
    seq = [
        cases.trsm_case("d", ColumnMajor, Left, Lower, NoTrans, NonUnit, 700, 300, alpha=1.5, pad=(3, 5), off=(2, 1), seed=31),
        cases.trsm_case("d", RowMajor, Right, Upper, Trans, Unit, 130, 260, alpha=-0.5, pad=(1, 2), off=(0, 3), seed=32),
        cases.trsm_case("d", ColumnMajor, Left, Upper, Trans, NonUnit, 129, 64, alpha=1.0, seed=33),
    ]
    for c in seq:
        logical = cases.trsm_logical(c)
        bufs = cases.trsm_buffers(c, logical)
        st, got = _run_noalloc(lib, c, bufs)
        assert st == lib.clblasSuccess, lib.STATUS_NAME.get(st, st)
        st2, want = run_trsm_gpu(lib, c, bufs)
        assert st2 == lib.clblasSuccess
        assert outside_untouched(bufs[1], got, c)
        X = oracle.view(got, c["order"], NoTrans, c["M"], c["N"], c["ldb"], c["offB"])
        Xw = oracle.view(want, c["order"], NoTrans, c["M"], c["N"], c["ldb"], c["offB"])
        n = c["M"] if c["side"] == Left else c["N"]
        # same tolerance as the TRSM parity tests use between two solutions of one system
        assert np.max(np.abs(X - Xw)) / (np.max(np.abs(Xw)) + 1e-30) <= 64 * n * oracle.unit_roundoff(np.float64)
        A, B = logical
        assert oracle.trsm_backward_ratio(X, c["alpha"], cases.trsm_op_triangle(c, A), B, c["side"], np.float64) <= 1.0
    assert lib.device_fault() == 0


def test_rejects_problems_beyond_the_scratch_array(lib):
    import torch
    n = lib.NOALLOC_MAX_ORDER + 1
    A = torch.ones(n * n, dtype=torch.float64, device="cuda")
    B = torch.ones(n * 4, dtype=torch.float64, device="cuda")
    before = B.clone()
    st = lib.clblasB200DtrsmNoAlloc(ColumnMajor, Left, Lower, NoTrans, NonUnit, n, 4, 1.0, A, 0, n, B, 0, n)
    assert st == lib.clblasOutOfResources
    wide = lib.NOALLOC_MAX_OTHER + 1
    B2 = torch.ones(8 * wide, dtype=torch.float64, device="cuda")
    st = lib.clblasB200DtrsmNoAlloc(ColumnMajor, Left, Lower, NoTrans, NonUnit, 8, wide, 1.0, A, 0, 8, B2, 0, 8)
    assert st == lib.clblasOutOfResources
    torch.cuda.synchronize()
    assert torch.equal(B, before)
