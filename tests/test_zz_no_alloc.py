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


def _big_lower_system(n, nrhs, offA, lda, offB, ldb, seed):
    """Left/Lower/NoTrans system generated on the device: diagonal in [1, 2], strict lower part U[-1, 1] / n, NaN above
    the diagonal and in every element of both buffers that does not belong to a matrix."""
    import torch
    g = torch.Generator(device="cuda")
    g.manual_seed(seed)
    A = torch.full((offA + lda * n,), float("nan"), dtype=torch.float64, device="cuda")
    Am = A[offA:].view(n, lda)[:, :n]                                  # Am[j, i] = A(i, j)
    Am.copy_(torch.empty(n, n, dtype=torch.float64, device="cuda").uniform_(-1.0, 1.0, generator=g) / n)
    Am.diagonal().uniform_(1.0, 2.0, generator=g)
    iu = torch.triu_indices(n, n, offset=1, device="cuda")
    Am[iu[1], iu[0]] = float("nan")
    B = torch.full((offB + ldb * nrhs,), float("nan"), dtype=torch.float64, device="cuda")
    B[offB:].view(nrhs, ldb)[:, :n].normal_(generator=g)
    return A, B


@pytest.mark.parametrize("n,nrhs,offA,pad_a,offB,pad_b", [
    (4096, 8192, 3, 1, 5, 3),        # exactly the limits; odd offsets and leading dimensions: the update products cannot use TMA
    (4096, 8192, 0, 0, 0, 0),        # exactly the limits, aligned: leaf products in place, updates with a partial last wave
    (2432, 8192, 0, 0, 0, 0),        # 19 diagonal blocks: odd splits, update grids of 5 x 64 ... 10 x 64 tiles (partial waves)
])
def test_allocates_nothing_up_to_the_limits(lib, n, nrhs, offA, pad_a, offB, pad_b):
    """The entry point is for callers who may not allocate, so the claim itself is checked: across a call the
    library's workspace-allocation counter must not move, for problems large enough that the ordinary DTRSM
    does allocate (inverted blocks; repacked operands for the unaligned case; stream-K partial tiles for update
    products with a partial last wave), and the result must be the ordinary DTRSM's."""
    import torch
    assert n <= lib.NOALLOC_MAX_ORDER and nrhs <= lib.NOALLOC_MAX_OTHER
    lda, ldb = n + pad_a, n + pad_b
    A, B0 = _big_lower_system(n, nrhs, offA, lda, offB, ldb, seed=41)
    args = (ColumnMajor, Left, Lower, NoTrans, NonUnit, n, nrhs, 1.0, A, offA, lda)
    lib.clblasB200DtrsmNoAlloc(ColumnMajor, Left, Lower, NoTrans, NonUnit, 8, 8, 1.0, A, offA, lda, B0.clone(), offB, ldb)   # one-time set-up
    torch.cuda.synchronize()
    X = B0.clone()
    before = lib.workspace_alloc_count()
    st = lib.clblasB200DtrsmNoAlloc(*args, X, offB, ldb)
    torch.cuda.synchronize()
    assert st == lib.clblasSuccess, lib.STATUS_NAME.get(st, st)
    assert lib.workspace_alloc_count() == before, "clblasB200DtrsmNoAlloc took a workspace"
    Y = B0.clone()
    st = lib.clblasDtrsm(*args, Y, offB, ldb)
    torch.cuda.synchronize()
    assert st == lib.clblasSuccess and lib.workspace_alloc_count() > before       # the ordinary entry point does allocate
    Xm, Ym = X[offB:].view(nrhs, ldb)[:, :n], Y[offB:].view(nrhs, ldb)[:, :n]
    assert bool(torch.isfinite(Xm).all())
    assert float((Xm - Ym).abs().max()) <= 64 * n * 2.0 ** -53 * float(Ym.abs().max())
    # padding and offset head untouched (NaN before and after)
    outside = torch.ones_like(X, dtype=torch.bool)
    outside[offB:].view(nrhs, ldb)[:, :n] = False
    assert bool(torch.isnan(X[outside]).all())
    # backward error of sampled columns on the host
    cols = np.unique(np.concatenate([np.random.Generator(np.random.Philox(key=[9, 1])).choice(nrhs, 20, replace=False), [0, nrhs - 1]]))
    ci = torch.from_numpy(cols).cuda()
    Xs, Bs = Xm[ci].cpu().numpy().T, B0[offB:].view(nrhs, ldb)[:, :n][ci].cpu().numpy().T
    T = np.tril(np.nan_to_num(A[offA:].view(n, lda)[:, :n].cpu().numpy().T, nan=0.0))
    assert oracle.trsm_backward_ratio(Xs, 1.0, T, Bs, Left, np.float64) <= 1.0
    assert lib.device_fault() == 0
