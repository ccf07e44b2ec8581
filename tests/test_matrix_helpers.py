"""Matrix helper API (clblasMatrixSizeInfo, clblas{Write,Read,Copy}{Sub,}Matrix, clblasFill*): host-side
logic on CPU, data movement on the GPU against numpy slicing.  Reference behaviour:
src/library/blas/matrix.c (region checks :27-47, row-major = x/y exchanged :240-262) and fill.cc."""
import ctypes

import numpy as np
import pytest

import clblas_b200 as cb

ROW, COL = cb.clblasRowMajor, cb.clblasColumnMajor


def test_matrix_size_info():
    # column-major: lines are columns of `rows` elements; row-major: lines are rows of `columns` elements
    assert cb.clblasMatrixSizeInfo(COL, 5, 7, 8, 3) == (cb.clblasSuccess, 8, 8 * 7 * 8)
    assert cb.clblasMatrixSizeInfo(ROW, 5, 7, 4, 1) == (cb.clblasSuccess, 8, 8 * 5 * 4)


def test_regions_outside_a_matrix_are_rejected_before_any_device_work():
    host = np.zeros(100, dtype=np.float32)
    fake_dev, q = 4096, 0
    sub = cb.lib.clblasWriteSubMatrix
    # 10 x 10 matrices; a 4 x 4 region at x = 8 leaves A
    assert sub(COL, 4, host.ctypes.data, 0, 10, 10, 10, 8, 0, fake_dev, 0, 10, 10, 10, 0, 0, 4, 4, q, 0, None) == cb.clblasInvalidValue
    # ... at y = 7 leaves B
    assert sub(COL, 4, host.ctypes.data, 0, 10, 10, 10, 0, 0, fake_dev, 0, 10, 10, 10, 0, 7, 4, 4, q, 0, None) == cb.clblasInvalidValue
    # row-major exchanges x and y: x = 8 is now the row position and 4 rows from row 8 leave the matrix
    assert sub(ROW, 4, host.ctypes.data, 0, 10, 10, 10, 8, 0, fake_dev, 0, 10, 10, 10, 0, 0, 4, 4, q, 0, None) == cb.clblasInvalidValue
    # leading dimension shorter than a line
    assert sub(COL, 4, host.ctypes.data, 0, 9, 10, 10, 0, 0, fake_dev, 0, 10, 10, 10, 0, 0, 4, 4, q, 0, None) == cb.clblasInvalidValue
    # a wait list without events
    assert cb.lib.clblasFillVector(4, 4, fake_dev, 0, ctypes.c_char_p(b"abcd"), q, 2, None) == cb.clblasInvalidEventWaitList


@pytest.mark.gpu
@pytest.mark.parametrize("order", [ROW, COL])
def test_write_read_copy_round_trip(lib, order):
    import torch
    rng = np.random.default_rng(5)
    rows, cols, lda, ldb = 37, 23, 41, 45
    inner, outer = (cols, rows) if order == ROW else (rows, cols)
    assert lda >= inner and ldb >= inner
    hostA = rng.standard_normal(3 + lda * outer).astype(np.float64)
    devB = torch.full((5 + ldb * outer,), float("nan"), dtype=torch.float64, device="cuda")
    assert cb.clblasWriteMatrix(order, rows, cols, 8, hostA, 3, lda, devB, 5, ldb) == cb.clblasSuccess
    A2 = hostA[3:].reshape(outer, lda)[:, :inner]
    B2 = devB.cpu().numpy()[5:].reshape(outer, ldb)
    assert np.array_equal(B2[:, :inner], A2) and np.all(np.isnan(B2[:, inner:]))
    # device -> device into a differently padded matrix, then back to the host
    devC = torch.zeros(lda * outer, dtype=torch.float64, device="cuda")
    assert cb.clblasCopyMatrix(order, rows, cols, 8, devB, 5, ldb, devC, 0, lda) == cb.clblasSuccess
    back = np.full(ldb * outer, -1.0)
    assert cb.clblasReadMatrix(order, rows, cols, 8, devC, 0, lda, back, 0, ldb) == cb.clblasSuccess
    assert np.array_equal(back.reshape(outer, ldb)[:, :inner], A2)
    assert np.all(back.reshape(outer, ldb)[:, inner:] == -1.0)


@pytest.mark.gpu
@pytest.mark.parametrize("order", [ROW, COL])
def test_sub_matrix_copies(lib, order):
    import torch
    rng = np.random.default_rng(6)
    nrA, ncA, nrB, ncB = 20, 30, 25, 40               # logical rows / columns
    A = rng.integers(-99, 99, size=(nrA, ncA)).astype(np.float32)
    B = np.zeros((nrB, ncB), dtype=np.float32)
    flatA = np.ascontiguousarray(A if order == ROW else A.T).reshape(-1)
    ldA, ldB = (ncA, ncB) if order == ROW else (nrA, nrB)
    devB = torch.zeros(nrB * ncB, dtype=torch.float32, device="cuda")
    xA, yA, xB, yB, nx, ny = 3, 5, 7, 11, 9, 13      # rows xA.., columns yA..: nx rows by ny columns
    st = cb.clblasWriteSubMatrix(order, 4, flatA, 0, ldA, nrA, ncA, xA, yA, devB, 0, ldB, nrB, ncB, xB, yB, nx, ny)
    assert st == cb.clblasSuccess
    B[xB:xB + nx, yB:yB + ny] = A[xA:xA + nx, yA:yA + ny]
    got = devB.cpu().numpy().reshape(nrB, ncB) if order == ROW else devB.cpu().numpy().reshape(ncB, nrB).T
    assert np.array_equal(got, B)
    # read a different window back
    out = np.zeros(nrA * ncA, dtype=np.float32)
    st = cb.clblasReadSubMatrix(order, 4, devB, 0, ldB, nrB, ncB, xB, yB, out, 0, ldA, nrA, ncA, 0, 0, nx, ny)
    assert st == cb.clblasSuccess
    outm = out.reshape(nrA, ncA) if order == ROW else out.reshape(ncA, nrA).T
    assert np.array_equal(outm[:nx, :ny], A[xA:xA + nx, yA:yA + ny])
    assert np.count_nonzero(outm) == np.count_nonzero(A[xA:xA + nx, yA:yA + ny])
    # an empty region succeeds and moves nothing
    assert cb.clblasCopySubMatrix(order, 4, devB, 0, ldB, nrB, ncB, 0, 0, devB, 0, ldB, nrB, ncB, 1, 1, 0, 5) == cb.clblasSuccess


@pytest.mark.gpu
def test_fills(lib):
    import torch
    d = torch.zeros(50 * 40, dtype=torch.float64, device="cuda")
    pat = np.array([2.5], dtype=np.float64).tobytes()
    assert cb.clblasFillSubMatrix(COL, 8, d, 0, 50, 50, 40, 5, 7, 10, 3, pat) == cb.clblasSuccess
    m = d.cpu().numpy().reshape(40, 50).T
    want = np.zeros((50, 40))
    want[5:15, 7:10] = 2.5
    assert np.array_equal(m, want)
    assert cb.clblasFillMatrix(ROW, 8, d, 0, 50, 40, 50, np.array([-1.0]).tobytes()) == cb.clblasSuccess
    assert torch.all(d == -1.0)
    # 16-byte elements (double complex), 4-byte elements at an offset, and a 12-byte pattern (byte path)
    z = torch.zeros(64, dtype=torch.complex128, device="cuda")
    assert cb.clblasFillVector(60, 16, z, 2, np.array([1 - 2j], dtype=np.complex128).tobytes()) == cb.clblasSuccess
    assert torch.all(z[2:62] == (1 - 2j)) and torch.all(z[:2] == 0) and torch.all(z[62:] == 0)
    f = torch.zeros(100, dtype=torch.float32, device="cuda")
    assert cb.clblasFillVector(10, 4, f, 3, np.array([7.0], dtype=np.float32).tobytes()) == cb.clblasSuccess
    assert torch.all(f[3:13] == 7.0) and f.sum().item() == 70.0
    t = torch.zeros(36, dtype=torch.float32, device="cuda")
    assert cb.clblasFillVector(3, 12, t, 0, np.array([1.0, 2.0, 3.0], dtype=np.float32).tobytes()) == cb.clblasSuccess
    assert t.cpu().numpy()[:9].tolist() == [1.0, 2.0, 3.0] * 3 and t[9:].sum().item() == 0.0


@pytest.mark.gpu
def test_create_matrix_from_host(lib):
    host = np.arange(12, dtype=np.float32)             # 3 x 4 row-major
    err = ctypes.c_int(-1)
    p = cb.lib.clblasCreateMatrixFromHost(None, ROW, 3, 4, 4, 6, host.ctypes.data, 0, 4, cb._stream(None), 0, None, ctypes.byref(err))
    assert err.value == 0 and p
    back = np.zeros(12, dtype=np.float32)
    assert cb.clblasReadMatrix(ROW, 3, 4, 4, p, 0, 6, back, 0, 4) == cb.clblasSuccess
    assert np.array_equal(back, host)
