"""Functional behaviour at the drop-in boundary on a real device, after the reference's functional
suite (src/tests/functional): error codes that need a device to decide (func-error.cpp:58-135),
events in and out (func-event.cpp:153-318), concurrent callers (func-thread.cpp:187-238), and the
check order of the GEMM / TRSM front ends (src/library/blas/xgemm.cc:685-706,
src/library/blas/functor/functor_xtrsm.cc:57-75)."""
import ctypes
import threading

import numpy as np
import pytest
import torch

import oracle
from oracle import ColumnMajor, Left, Lower, NonUnit, NoTrans, RowMajor, Trans
from tests import cases
from tests.gpu_util import dev

pytestmark = pytest.mark.gpu


def test_gemm_error_codes(lib):
    n = 256
    A = torch.ones(n * n, dtype=torch.float32, device="cuda")
    B = torch.ones(n * n, dtype=torch.float32, device="cuda")
    C = torch.zeros(n * n, dtype=torch.float32, device="cuda")
    ok = (lib.clblasColumnMajor, lib.clblasNoTrans, lib.clblasNoTrans, n, n, n, 1.0)
    assert lib.clblasSgemm(*ok, A, 0, n, B, 0, n, 0.0, C, 0, n) == lib.clblasSuccess
    # leading dimensions: lda < M (column-major, NoTrans), ldb < K, ldc < M
    assert lib.clblasSgemm(*ok, A, 0, n - 1, B, 0, n, 0.0, C, 0, n) == lib.clblasInvalidLeadDimA
    assert lib.clblasSgemm(*ok, A, 0, n, B, 0, n - 1, 0.0, C, 0, n) == lib.clblasInvalidLeadDimB
    assert lib.clblasSgemm(*ok, A, 0, n, B, 0, n, 0.0, C, 0, n - 1) == lib.clblasInvalidLeadDimC
    # row-major, transposed A: lda must be >= M
    assert lib.clblasSgemm(lib.clblasRowMajor, lib.clblasTrans, lib.clblasNoTrans, n, n, 8, 1.0, A, 0, n - 1, B, 0, n,
                           0.0, C, 0, n) == lib.clblasInvalidLeadDimA
    # zero dimensions (generic/common.c:601-603)
    assert lib.clblasSgemm(lib.clblasColumnMajor, 0, 0, 0, n, n, 1.0, A, 0, n, B, 0, n, 0.0, C, 0, n) == lib.clblasInvalidDim
    assert lib.clblasSgemm(lib.clblasColumnMajor, 0, 0, n, 0, n, 1.0, A, 0, n, B, 0, n, 0.0, C, 0, n) == lib.clblasInvalidDim
    # a host address is not a device buffer
    host = np.ones(n * n, dtype=np.float32)
    assert lib.clblasSgemm(*ok, host.ctypes.data, 0, n, B, 0, n, 0.0, C, 0, n) in (lib.clblasInvalidMatA, lib.clblasInsufficientMemMatA)
    # queue and event list checks
    none = ctypes.POINTER(ctypes.c_void_p)()
    raw = lib.lib.clblasSgemm
    args = (1, 0, 0, n, n, n, 1.0, A.data_ptr(), 0, n, B.data_ptr(), 0, n, 0.0, C.data_ptr(), 0, n)
    assert raw(*args, 0, none, 0, none, none) == lib.clblasInvalidCommandQueue
    q = (ctypes.c_void_p * 1)(torch.cuda.current_stream().cuda_stream)
    assert raw(*args, 1, q, 1, none, none) == lib.clblasInvalidEventWaitList
    torch.cuda.synchronize()


def test_insufficient_memory_is_detected(lib):
    """The reference doubles the sizes against the buffers it created and expects
    clblasInsufficientMemMatA (func-error.cpp:86-101).  Buffers of 64 MiB each, so that the caching
    allocator's block is the tensor itself, asked for four times their extent."""
    n = 4096
    torch.cuda.synchronize()
    torch.cuda.empty_cache()             # fresh driver allocations, not slices of a larger cached block
    A = torch.empty(n * n, dtype=torch.float32, device="cuda")
    B = torch.empty(n * n, dtype=torch.float32, device="cuda")
    C = torch.empty(n * n, dtype=torch.float32, device="cuda")
    big = 2 * n
    st = lib.clblasSgemm(lib.clblasColumnMajor, lib.clblasNoTrans, lib.clblasNoTrans, big, n, big, 1.0, A, 0, big, B, 0, big,
                         0.0, C, 0, big)
    assert st == lib.clblasInsufficientMemMatA
    st = lib.clblasSgemm(lib.clblasColumnMajor, lib.clblasNoTrans, lib.clblasNoTrans, n, big, n, 1.0, A, 0, n, B, 0, n,
                         0.0, C, 0, n)
    assert st == lib.clblasInsufficientMemMatB
    st = lib.clblasSgemm(lib.clblasColumnMajor, lib.clblasNoTrans, lib.clblasNoTrans, n, n, n, 1.0, A, 0, n, B, 0, n,
                         0.0, C, n * n, n)
    assert st == lib.clblasInsufficientMemMatC
    st = lib.clblasDtrsm(lib.clblasColumnMajor, lib.clblasLeft, lib.clblasLower, lib.clblasNoTrans, lib.clblasNonUnit,
                         n, n, 1.0, A, 0, n, B, 0, n)               # float buffers are half the size a double solve needs
    assert st == lib.clblasInsufficientMemMatA


def test_trsm_needs_setup_and_checks_in_reference_order(lib):
    A = torch.eye(64, dtype=torch.float64, device="cuda").reshape(-1).contiguous()
    B = torch.ones(64 * 8, dtype=torch.float64, device="cuda")
    args = (lib.clblasColumnMajor, lib.clblasLeft, lib.clblasLower, lib.clblasNoTrans, lib.clblasNonUnit, 64, 8, 1.0)
    lib.clblasTeardown()
    try:
        assert lib.clblasDtrsm(*args, A, 0, 64, B, 0, 64) == lib.clblasNotInitialized
        # GEMM does not depend on Setup in the reference either (AutoGemm path)
        C = torch.zeros(64 * 64, dtype=torch.float64, device="cuda")
        assert lib.clblasDgemm(lib.clblasColumnMajor, 0, 0, 64, 64, 64, 1.0, A, 0, 64, A, 0, 64, 0.0, C, 0, 64) == lib.clblasSuccess
    finally:
        assert lib.clblasSetup() == lib.clblasSuccess
    assert lib.clblasDtrsm(*args, None, 0, 64, B, 0, 64) == lib.clblasInvalidMatA
    assert lib.clblasDtrsm(*args, A, 0, 64, None, 0, 64) == lib.clblasInvalidMatB
    assert lib.clblasDtrsm(*args, A, 0, 63, B, 0, 64) == lib.clblasInvalidLeadDimA
    assert lib.clblasDtrsm(*args, A, 0, 64, B, 0, 63) == lib.clblasInvalidLeadDimB
    assert lib.clblasDtrsm(lib.clblasColumnMajor, lib.clblasLeft, lib.clblasLower, 0, 1, 0, 8, 1.0, A, 0, 64, B, 0, 64) == lib.clblasInvalidDim
    assert lib.clblasDtrsm(*args, A, 0, 64, B, 0, 64) == lib.clblasSuccess
    torch.cuda.synchronize()
    assert torch.all(B == 1.0)


def test_events_in_and_out(lib):
    """EVENT_IN: the call must not start before the events of its wait list; EVENT_OUT: the returned
    event completes when the result is ready (func-event.cpp:153-318)."""
    n = 1024
    c = cases.gemm_case("d", ColumnMajor, NoTrans, NoTrans, n, n, n, alpha=1.0, beta=0.0, mode="int")
    opA, opB, C0 = cases.gemm_logical(c)
    hA, hB, hC = cases.gemm_buffers(c, (opA, opB, C0), tail=0)
    dA = torch.empty(hA.size, dtype=torch.float64, device="cuda")
    dB, dC = dev(hB), dev(hC)
    producer, consumer = torch.cuda.Stream(), torch.cuda.Stream()
    ready, done = torch.cuda.Event(), torch.cuda.Event()
    pinned = torch.from_numpy(hA).pin_memory()
    with torch.cuda.stream(producer):
        torch.cuda._sleep(50_000_000)                    # keep A's upload pending for a while
        dA.copy_(pinned, non_blocking=True)
        ready.record(producer)
    done.record(consumer)                                # create the handle; re-recorded by the library
    st = lib.clblasDgemm(c["order"], c["transA"], c["transB"], n, n, n, 1.0, dA, 0, c["lda"], dB, 0, c["ldb"], 0.0, dC, 0, c["ldc"],
                         queues=[consumer], wait=[ready], events=[done])
    assert st == lib.clblasSuccess
    done.synchronize()                                   # EVENT_OUT: nothing else is synchronised
    got = dC.cpu().numpy()
    want = (opA @ opB).astype(np.float64)
    assert np.array_equal(oracle.view(got, ColumnMajor, NoTrans, n, n, c["ldc"], 0), want)
    torch.cuda.synchronize()


def test_concurrent_host_threads(lib):
    """The entry points are thread safe (src/clBLAS.h:59-61, func-thread.cpp:187-238): several host
    threads, each with its own stream and buffers, mixing GEMM and TRSM."""
    results, errors = {}, []

    def worker(k):
        try:
            torch.cuda.set_device(0)
            s = torch.cuda.Stream()
            prec = "sd"[k % 2]
            c = cases.gemm_case(prec, ColumnMajor, [NoTrans, Trans][k % 2], NoTrans, 192 + 8 * k, 160, 200 + k, alpha=2.0, beta=1.0,
                                mode="int", seed=900 + k)
            opA, opB, C0 = cases.gemm_logical(c)
            hA, hB, hC = cases.gemm_buffers(c, (opA, opB, C0))
            with torch.cuda.stream(s):
                dA, dB, dC = dev(hA), dev(hB), dev(hC)
                fn = lib.clblasSgemm if prec == "s" else lib.clblasDgemm
                for _ in range(5):
                    dC.copy_(torch.from_numpy(hC))
                    st = fn(c["order"], c["transA"], c["transB"], c["M"], c["N"], c["K"], 2.0, dA, 0, c["lda"], dB, 0, c["ldb"], 1.0,
                            dC, 0, c["ldc"], queues=[s])
                    assert st == lib.clblasSuccess
                t = cases.trsm_case("d", ColumnMajor, Left, Lower, NoTrans, NonUnit, 200 + k, 96, seed=950 + k)
                TA, TB = cases.trsm_logical(t)
                tA, tB = cases.trsm_buffers(t, (TA, TB))
                dTA, dTB = dev(tA), dev(tB)
                assert lib.clblasDtrsm(t["order"], t["side"], t["uplo"], t["transA"], t["diag"], t["M"], t["N"], 1.0, dTA, 0, t["lda"],
                                       dTB, 0, t["ldb"], queues=[s]) == lib.clblasSuccess
            s.synchronize()
            want = (2.0 * (opA.astype(np.float64) @ opB.astype(np.float64)) + C0).astype(cases.DT[prec])
            ok_gemm = np.array_equal(oracle.view(dC.cpu().numpy(), ColumnMajor, NoTrans, c["M"], c["N"], c["ldc"], 0), want)
            X = oracle.view(dTB.cpu().numpy(), ColumnMajor, NoTrans, t["M"], t["N"], t["ldb"], 0)
            ok_trsm = oracle.trsm_backward_ratio(X, 1.0, cases.trsm_op_triangle(t, TA), TB, Left, np.float64) <= 1.0
            results[k] = (ok_gemm, ok_trsm)
        except Exception as e:  # noqa: BLE001
            errors.append((k, repr(e)))

    threads = [threading.Thread(target=worker, args=(k,)) for k in range(6)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors
    assert len(results) == 6 and all(a and b for a, b in results.values()), results
    assert lib.device_fault() == 0
