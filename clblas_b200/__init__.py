"""clblas_b200 -- host-side mirror of the clBLAS level-3 entry points over the B200 C-ABI library.

The functions keep the reference's names, argument order and status-code convention
(src/clBLAS.h:7382-7405 clblasSgemm, :7463-7486 clblasDgemm, :7988-8008 clblasStrsm,
:8063-8083 clblasDtrsm): they return a ``clblasStatus`` integer and raise nothing on a bad
argument.  Buffers are CUDA device pointers (a ``torch.Tensor`` on a CUDA device or a raw
integer address); queues are CUDA streams; events are CUDA events.

All work is done by ``lib/libclblas_b200.so`` (hand-written sm_100a kernels behind
``include/clblas_b200.h``).  There is no CPU path: importing this package without the built
library raises ``ImportError``.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional, Sequence

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libclblas_b200.so")

# enums (src/clBLAS.h:78-113)
clblasRowMajor, clblasColumnMajor = 0, 1
clblasNoTrans, clblasTrans, clblasConjTrans = 0, 1, 2
clblasUpper, clblasLower = 0, 1
clblasUnit, clblasNonUnit = 0, 1
clblasLeft, clblasRight = 0, 1

# status codes (src/clBLAS.h:123-155)
STATUS = {
    "clblasSuccess": 0, "clblasInvalidValue": -30, "clblasInvalidCommandQueue": -36,
    "clblasInvalidContext": -34, "clblasInvalidMemObject": -38, "clblasInvalidDevice": -33,
    "clblasInvalidEventWaitList": -57, "clblasOutOfResources": -5, "clblasOutOfHostMemory": -6,
    "clblasInvalidOperation": -59, "clblasCompilerNotAvailable": -3, "clblasBuildProgramFailure": -11,
    "clblasNotImplemented": -1024, "clblasNotInitialized": -1023, "clblasInvalidMatA": -1022,
    "clblasInvalidMatB": -1021, "clblasInvalidMatC": -1020, "clblasInvalidVecX": -1019,
    "clblasInvalidVecY": -1018, "clblasInvalidDim": -1017, "clblasInvalidLeadDimA": -1016,
    "clblasInvalidLeadDimB": -1015, "clblasInvalidLeadDimC": -1014, "clblasInvalidIncX": -1013,
    "clblasInvalidIncY": -1012, "clblasInsufficientMemMatA": -1011, "clblasInsufficientMemMatB": -1010,
    "clblasInsufficientMemMatC": -1009, "clblasInsufficientMemVecX": -1008, "clblasInsufficientMemVecY": -1007,
}
globals().update(STATUS)
STATUS_NAME = {v: k for k, v in STATUS.items()}


class ClblasError(RuntimeError):
    def __init__(self, status: int, what: str = ""):
        self.status = status
        super().__init__(f"{what}: {STATUS_NAME.get(status, status)} ({status})")


def check(status: int, what: str = "clblas call") -> None:
    """Raise ClblasError unless status is clblasSuccess (convenience; the entry points never raise)."""
    if status != 0:
        raise ClblasError(status, what)


class FloatComplex(ctypes.Structure):
    """(re, im) pair passed by value, layout of the reference's FloatComplex (cl_float2)."""
    _fields_ = [("re", ctypes.c_float), ("im", ctypes.c_float)]


class DoubleComplex(ctypes.Structure):
    _fields_ = [("re", ctypes.c_double), ("im", ctypes.c_double)]


MATRIX_HELPERS = (["clblasMatrixSizeInfo", "clblasCreateMatrix", "clblasCreateMatrixWithLd", "clblasCreateMatrixFromHost",
                   "clblasFillVector", "clblasFillVectorAsync", "clblasFillSubMatrix", "clblasFillSubMatrixAsync",
                   "clblasFillMatrix", "clblasFillMatrixAsync"]
                  + [f"clblas{k}{s}Matrix{a}" for k in ("Write", "Read", "Copy") for s in ("Sub", "") for a in ("", "Async")])


COMPLEX_SYM = [f"clblas{p}{r}" for p in "CZ" for r in ("syrk", "herk", "syr2k", "her2k", "symm", "hemm")]


def _load() -> ctypes.CDLL:
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python clblas_b200/build.py` "
            "(there is no CPU or PyTorch fallback for these routines)")
    lib = ctypes.CDLL(LIB_PATH)
    sz, u, i, vp = ctypes.c_size_t, ctypes.c_uint, ctypes.c_int, ctypes.c_void_p
    pvp = ctypes.POINTER(ctypes.c_void_p)
    for name, ft in (("clblasSgemm", ctypes.c_float), ("clblasDgemm", ctypes.c_double),
                     ("clblasB200SgemmHost", ctypes.c_float), ("clblasB200DgemmHost", ctypes.c_double)):
        f = getattr(lib, name)
        f.argtypes = [i, i, i, sz, sz, sz, ft, vp, sz, sz, vp, sz, sz, ft, vp, sz, sz, u, pvp, u, pvp, pvp]
        f.restype = i
    for name, ft in (("clblasStrsm", ctypes.c_float), ("clblasDtrsm", ctypes.c_double),
                     ("clblasB200DtrsmNoAlloc", ctypes.c_double), ("clblasStrmm", ctypes.c_float),
                     ("clblasB200StrsmHost", ctypes.c_float), ("clblasB200DtrsmHost", ctypes.c_double),
                     ("clblasDtrmm", ctypes.c_double)):
        f = getattr(lib, name)
        f.argtypes = [i, i, i, i, i, sz, sz, ft, vp, sz, sz, vp, sz, sz, u, pvp, u, pvp, pvp]
        f.restype = i
    for name, ft in (("clblasSsyrk", ctypes.c_float), ("clblasDsyrk", ctypes.c_double)):
        f = getattr(lib, name)
        f.argtypes = [i, i, i, sz, sz, ft, vp, sz, sz, ft, vp, sz, sz, u, pvp, u, pvp, pvp]
        f.restype = i
    for name, ft in (("clblasSsyr2k", ctypes.c_float), ("clblasDsyr2k", ctypes.c_double)):
        f = getattr(lib, name)
        f.argtypes = [i, i, i, sz, sz, ft, vp, sz, sz, vp, sz, sz, ft, vp, sz, sz, u, pvp, u, pvp, pvp]
        f.restype = i
    for name, ft in (("clblasSsymm", ctypes.c_float), ("clblasDsymm", ctypes.c_double)):
        f = getattr(lib, name)
        f.argtypes = [i, i, i, sz, sz, ft, vp, sz, sz, vp, sz, sz, ft, vp, sz, sz, u, pvp, u, pvp, pvp]
        f.restype = i
    for name, ct in (("clblasCgemm", FloatComplex), ("clblasZgemm", DoubleComplex)):
        f = getattr(lib, name)
        f.argtypes = [i, i, i, sz, sz, sz, ct, vp, sz, sz, vp, sz, sz, ct, vp, sz, sz, u, pvp, u, pvp, pvp]
        f.restype = i
    for name, ct in (("clblasCtrsm", FloatComplex), ("clblasZtrsm", DoubleComplex), ("clblasCtrmm", FloatComplex),
                     ("clblasZtrmm", DoubleComplex)):
        f = getattr(lib, name)
        f.argtypes = [i, i, i, i, i, sz, sz, ct, vp, sz, sz, vp, sz, sz, u, pvp, u, pvp, pvp]
        f.restype = i
    # matrix helpers (one stream, not an array of queues)
    psz, pint = ctypes.POINTER(sz), ctypes.POINTER(i)
    lib.clblasMatrixSizeInfo.argtypes = [i, sz, sz, sz, sz, psz, psz]
    lib.clblasCreateMatrix.argtypes = [vp, i, sz, sz, sz, sz, psz, psz, pint]
    lib.clblasCreateMatrixWithLd.argtypes = [vp, i, sz, sz, sz, sz, psz, pint]
    lib.clblasCreateMatrixFromHost.argtypes = [vp, i, sz, sz, sz, sz, vp, sz, sz, vp, u, pvp, pint]
    for name in ("clblasCreateMatrix", "clblasCreateMatrixWithLd", "clblasCreateMatrixFromHost"):
        getattr(lib, name).restype = vp
    sub = [i, sz, vp, sz, sz, sz, sz, sz, sz, vp, sz, sz, sz, sz, sz, sz, sz, sz, vp, u, pvp]
    full = [i, sz, sz, sz, vp, sz, sz, vp, sz, sz, vp, u, pvp]
    for kind in ("Write", "Read", "Copy"):
        getattr(lib, f"clblas{kind}SubMatrix").argtypes = sub
        getattr(lib, f"clblas{kind}SubMatrixAsync").argtypes = sub + [pvp]
        getattr(lib, f"clblas{kind}Matrix").argtypes = full
        getattr(lib, f"clblas{kind}MatrixAsync").argtypes = full + [pvp]
    lib.clblasFillVector.argtypes = [sz, sz, vp, sz, vp, vp, u, pvp]
    lib.clblasFillVectorAsync.argtypes = lib.clblasFillVector.argtypes + [pvp]
    lib.clblasFillSubMatrix.argtypes = [i, sz, vp, sz, sz, sz, sz, sz, sz, sz, sz, vp, vp, u, pvp]
    lib.clblasFillSubMatrixAsync.argtypes = lib.clblasFillSubMatrix.argtypes + [pvp]
    lib.clblasFillMatrix.argtypes = [i, sz, vp, sz, sz, sz, sz, vp, vp, u, pvp]
    lib.clblasFillMatrixAsync.argtypes = lib.clblasFillMatrix.argtypes + [pvp]
    for name in MATRIX_HELPERS:
        if not name.startswith("clblasCreate"):
            getattr(lib, name).restype = i
    tail = [u, pvp, u, pvp, pvp]
    for name, ct, rt in (("clblasCsyrk", FloatComplex, None), ("clblasZsyrk", DoubleComplex, None),
                         ("clblasCherk", None, ctypes.c_float), ("clblasZherk", None, ctypes.c_double)):
        a = ct or rt
        getattr(lib, name).argtypes = [i, i, i, sz, sz, a, vp, sz, sz, a, vp, sz, sz] + tail
        getattr(lib, name).restype = i
    for name, ct, bt in (("clblasCsyr2k", FloatComplex, FloatComplex), ("clblasZsyr2k", DoubleComplex, DoubleComplex),
                         ("clblasCher2k", FloatComplex, ctypes.c_float), ("clblasZher2k", DoubleComplex, ctypes.c_double)):
        getattr(lib, name).argtypes = [i, i, i, sz, sz, ct, vp, sz, sz, vp, sz, sz, bt, vp, sz, sz] + tail
        getattr(lib, name).restype = i
    for name, ct in (("clblasCsymm", FloatComplex), ("clblasZsymm", DoubleComplex), ("clblasChemm", FloatComplex),
                     ("clblasZhemm", DoubleComplex)):
        getattr(lib, name).argtypes = [i, i, i, sz, sz, ct, vp, sz, sz, vp, sz, sz, ct, vp, sz, sz] + tail
        getattr(lib, name).restype = i
    lib.clblasSetup.argtypes = []
    lib.clblasSetup.restype = i
    lib.clblasTeardown.argtypes = []
    lib.clblasTeardown.restype = None
    lib.clblasGetVersion.argtypes = [ctypes.POINTER(u)] * 3
    lib.clblasGetVersion.restype = i
    lib.clblasB200PlanShards.argtypes = [sz, u, sz, ctypes.POINTER(sz)]
    lib.clblasB200PlanShards.restype = i
    lib.clblasB200LaunchCount.argtypes = []
    lib.clblasB200LaunchCount.restype = ctypes.c_ulonglong
    lib.clblasB200ProbePeak.argtypes = [i, ctypes.c_double]
    lib.clblasB200ProbePeak.restype = ctypes.c_double
    lib.clblasB200DeviceFault.argtypes = []
    lib.clblasB200DeviceFault.restype = ctypes.c_uint
    lib.clblasB200LastGemmKernel.argtypes = []
    lib.clblasB200LastGemmKernel.restype = ctypes.c_char_p
    lib.clblasB200SetGemmPath.argtypes = [i]
    lib.clblasB200SetGemmPath.restype = i
    lib.clblasB200LastGemmVariant.argtypes = []
    lib.clblasB200LastGemmVariant.restype = ctypes.c_char_p
    lib.clblasB200WorkspaceAllocCount.argtypes = []
    lib.clblasB200WorkspaceAllocCount.restype = ctypes.c_ulonglong
    lib.clblasB200NoAllocLimits.argtypes = [psz, psz]
    lib.clblasB200NoAllocLimits.restype = None
    # communicator and sharded forms
    lib.clblasB200CommGetUniqueId.argtypes = [vp]
    lib.clblasB200CommInitRank.argtypes = [pvp, vp, i, i]
    lib.clblasB200CommInitAll.argtypes = [pvp, i, pint]
    lib.clblasB200CommDestroy.argtypes = [vp]
    lib.clblasB200CommInfo.argtypes = [vp, pint, pint]
    lib.clblasB200PanelPlan.argtypes = [sz, sz, u, psz, ctypes.POINTER(u)]
    for name in ("clblasB200CommGetUniqueId", "clblasB200CommInitRank", "clblasB200CommInitAll", "clblasB200CommDestroy",
                 "clblasB200CommInfo", "clblasB200PanelPlan"):
        getattr(lib, name).restype = i
    for name, ft in (("clblasB200SgemmSharded", ctypes.c_float), ("clblasB200DgemmSharded", ctypes.c_double)):
        f = getattr(lib, name)
        f.argtypes = [i, i, i, sz, sz, sz, ft, vp, sz, sz, vp, sz, sz, ft, vp, sz, sz, vp, i, u, pvp, u, pvp, pvp]
        f.restype = i
    for name, ft in (("clblasB200StrsmSharded", ctypes.c_float), ("clblasB200DtrsmSharded", ctypes.c_double)):
        f = getattr(lib, name)
        f.argtypes = [i, i, i, i, i, sz, sz, ft, vp, sz, sz, vp, sz, sz, vp, i, u, pvp, u, pvp, pvp]
        f.restype = i
    return lib


lib = _load()

EXPORTS = ["clblasSetup", "clblasTeardown", "clblasGetVersion", "clblasSgemm", "clblasDgemm", "clblasStrsm",
           "clblasDtrsm", "clblasB200PlanShards", "clblasB200LaunchCount", "clblasB200LastGemmKernel",
           "clblasB200SetGemmPath", "clblasB200DeviceFault", "clblasB200ProbePeak", "clblasB200DtrsmNoAlloc",
           "clblasStrmm", "clblasDtrmm", "clblasSsyrk", "clblasDsyrk", "clblasSsyr2k", "clblasDsyr2k",
           "clblasSsymm", "clblasDsymm", "clblasCgemm", "clblasZgemm", "clblasCtrsm", "clblasZtrsm", "clblasB200SgemmHost", "clblasB200DgemmHost", "clblasB200StrsmHost", "clblasB200DtrsmHost"] + MATRIX_HELPERS + COMPLEX_SYM + ["clblasCtrmm", "clblasZtrmm"] + [
    "clblasB200LastGemmVariant", "clblasB200WorkspaceAllocCount", "clblasB200NoAllocLimits", "clblasB200CommGetUniqueId",
    "clblasB200CommInitRank", "clblasB200CommInitAll", "clblasB200CommDestroy", "clblasB200CommInfo", "clblasB200PanelPlan",
    "clblasB200SgemmSharded", "clblasB200DgemmSharded", "clblasB200StrsmSharded", "clblasB200DtrsmSharded"]


def _ptr(x) -> Optional[int]:
    if x is None:
        return None
    if isinstance(x, int):
        return x
    return x.data_ptr()      # torch.Tensor


def _handle(x) -> Optional[int]:
    """CUDA stream / event handle from a torch object or a raw integer."""
    if x is None:
        return None
    if isinstance(x, int):
        return x
    for attr in ("cuda_stream", "cuda_event"):
        if hasattr(x, attr):
            return getattr(x, attr)
    raise TypeError(f"not a CUDA stream or event: {x!r}")


def _handle_array(items: Optional[Sequence], default_current_stream: bool = False):
    if items is None:
        if not default_current_stream:
            return 0, None
        import torch
        items = [torch.cuda.current_stream()]
    arr = (ctypes.c_void_p * max(len(items), 1))()
    for k, it in enumerate(items):
        arr[k] = _handle(it)
    return len(items), arr


def _queues_events(queues, wait, events):
    nq, q = _handle_array(queues, default_current_stream=True)
    nw, w = _handle_array(wait)
    _, e = _handle_array(events)
    return nq, q, nw, w, e


def clblasSetup() -> int:
    return lib.clblasSetup()


def clblasTeardown() -> None:
    lib.clblasTeardown()


def clblasGetVersion():
    a, b, c = ctypes.c_uint(), ctypes.c_uint(), ctypes.c_uint()
    st = lib.clblasGetVersion(ctypes.byref(a), ctypes.byref(b), ctypes.byref(c))
    return st, (a.value, b.value, c.value)


def _gemm(fn, order, transA, transB, M, N, K, alpha, A, offA, lda, B, offB, ldb, beta, C, offC, ldc,
          queues, wait, events):
    nq, q, nw, w, e = _queues_events(queues, wait, events)
    return fn(order, transA, transB, M, N, K, alpha, _ptr(A), offA, lda, _ptr(B), offB, ldb, beta,
              _ptr(C), offC, ldc, nq, q, nw, w, e)


def clblasSgemm(order, transA, transB, M, N, K, alpha, A, offA, lda, B, offB, ldb, beta, C, offC, ldc,
                queues=None, wait=None, events=None) -> int:
    """float GEMM; `queues` defaults to torch's current stream, like passing one command queue."""
    return _gemm(lib.clblasSgemm, order, transA, transB, M, N, K, alpha, A, offA, lda, B, offB, ldb, beta,
                 C, offC, ldc, queues, wait, events)


def clblasDgemm(order, transA, transB, M, N, K, alpha, A, offA, lda, B, offB, ldb, beta, C, offC, ldc,
                queues=None, wait=None, events=None) -> int:
    return _gemm(lib.clblasDgemm, order, transA, transB, M, N, K, alpha, A, offA, lda, B, offB, ldb, beta,
                 C, offC, ldc, queues, wait, events)


def _host_addr(x) -> Optional[int]:
    """Address of a host matrix: a numpy array, a CPU torch tensor or a raw integer."""
    if x is None or isinstance(x, int):
        return x
    if hasattr(x, "data_ptr"):
        if getattr(x, "is_cuda", False):
            raise TypeError("host GEMM takes host memory; use clblasSgemm / clblasDgemm for device tensors")
        return x.data_ptr()
    return x.ctypes.data


def _gemm_host(fn, order, transA, transB, M, N, K, alpha, A, offA, lda, B, offB, ldb, beta, C, offC, ldc, queues, wait, events):
    nq, q, nw, w, e = _queues_events(queues, wait, events)
    return fn(order, transA, transB, M, N, K, alpha, _host_addr(A), offA, lda, _host_addr(B), offB, ldb, beta,
              _host_addr(C), offC, ldc, nq, q, nw, w, e)


def clblasB200SgemmHost(order, transA, transB, M, N, K, alpha, A, offA, lda, B, offB, ldb, beta, C, offC, ldc,
                        queues=None, wait=None, events=None) -> int:
    """float GEMM on HOST matrices (numpy arrays or CPU tensors, pinned for speed): uploads, products and downloads
    overlap.  The result is in C once the stream (default: torch's current stream) has completed."""
    return _gemm_host(lib.clblasB200SgemmHost, order, transA, transB, M, N, K, alpha, A, offA, lda, B, offB, ldb, beta,
                      C, offC, ldc, queues, wait, events)


def clblasB200DgemmHost(order, transA, transB, M, N, K, alpha, A, offA, lda, B, offB, ldb, beta, C, offC, ldc,
                        queues=None, wait=None, events=None) -> int:
    return _gemm_host(lib.clblasB200DgemmHost, order, transA, transB, M, N, K, alpha, A, offA, lda, B, offB, ldb, beta,
                      C, offC, ldc, queues, wait, events)


def _trsm_host(fn, order, side, uplo, transA, diag, M, N, alpha, A, offA, lda, B, offB, ldb, queues, wait, events):
    nq, q, nw, w, e = _queues_events(queues, wait, events)
    return fn(order, side, uplo, transA, diag, M, N, alpha, _host_addr(A), offA, lda, _host_addr(B), offB, ldb, nq, q, nw, w, e)


def clblasB200StrsmHost(order, side, uplo, transA, diag, M, N, alpha, A, offA, lda, B, offB, ldb,
                        queues=None, wait=None, events=None) -> int:
    """float TRSM on HOST matrices: blocks of right-hand sides uploaded, solved and downloaded in a pipeline."""
    return _trsm_host(lib.clblasB200StrsmHost, order, side, uplo, transA, diag, M, N, alpha, A, offA, lda, B, offB, ldb,
                      queues, wait, events)


def clblasB200DtrsmHost(order, side, uplo, transA, diag, M, N, alpha, A, offA, lda, B, offB, ldb,
                        queues=None, wait=None, events=None) -> int:
    return _trsm_host(lib.clblasB200DtrsmHost, order, side, uplo, transA, diag, M, N, alpha, A, offA, lda, B, offB, ldb,
                      queues, wait, events)


def _trsm(fn, order, side, uplo, transA, diag, M, N, alpha, A, offA, lda, B, offB, ldb, queues, wait, events):
    nq, q, nw, w, e = _queues_events(queues, wait, events)
    return fn(order, side, uplo, transA, diag, M, N, alpha, _ptr(A), offA, lda, _ptr(B), offB, ldb,
              nq, q, nw, w, e)


def clblasStrsm(order, side, uplo, transA, diag, M, N, alpha, A, offA, lda, B, offB, ldb,
                queues=None, wait=None, events=None) -> int:
    return _trsm(lib.clblasStrsm, order, side, uplo, transA, diag, M, N, alpha, A, offA, lda, B, offB, ldb,
                 queues, wait, events)


def clblasDtrsm(order, side, uplo, transA, diag, M, N, alpha, A, offA, lda, B, offB, ldb,
                queues=None, wait=None, events=None) -> int:
    return _trsm(lib.clblasDtrsm, order, side, uplo, transA, diag, M, N, alpha, A, offA, lda, B, offB, ldb,
                 queues, wait, events)


def clblasStrmm(order, side, uplo, transA, diag, M, N, alpha, A, offA, lda, B, offB, ldb,
                queues=None, wait=None, events=None) -> int:
    """B <- alpha*op(A)*B (Left) / alpha*B*op(A) (Right), A triangular (src/clBLAS.h:7697-7717)."""
    return _trsm(lib.clblasStrmm, order, side, uplo, transA, diag, M, N, alpha, A, offA, lda, B, offB, ldb,
                 queues, wait, events)


def clblasDtrmm(order, side, uplo, transA, diag, M, N, alpha, A, offA, lda, B, offB, ldb,
                queues=None, wait=None, events=None) -> int:
    return _trsm(lib.clblasDtrmm, order, side, uplo, transA, diag, M, N, alpha, A, offA, lda, B, offB, ldb,
                 queues, wait, events)


def _syrk(fn, order, uplo, transA, N, K, alpha, A, offA, lda, beta, C, offC, ldc, queues, wait, events):
    nq, q, nw, w, e = _queues_events(queues, wait, events)
    return fn(order, uplo, transA, N, K, alpha, _ptr(A), offA, lda, beta, _ptr(C), offC, ldc, nq, q, nw, w, e)


def clblasSsyrk(order, uplo, transA, N, K, alpha, A, offA, lda, beta, C, offC, ldc, queues=None, wait=None, events=None) -> int:
    """C <- alpha*op(A)*op(A)^T + beta*C on one triangle of C (src/clBLAS.h:8279-8296)."""
    return _syrk(lib.clblasSsyrk, order, uplo, transA, N, K, alpha, A, offA, lda, beta, C, offC, ldc, queues, wait, events)


def clblasDsyrk(order, uplo, transA, N, K, alpha, A, offA, lda, beta, C, offC, ldc, queues=None, wait=None, events=None) -> int:
    return _syrk(lib.clblasDsyrk, order, uplo, transA, N, K, alpha, A, offA, lda, beta, C, offC, ldc, queues, wait, events)


def _abc(fn, e0, e1, e2, d0, d1, alpha, A, offA, lda, B, offB, ldb, beta, C, offC, ldc, queues, wait, events):
    nq, q, nw, w, e = _queues_events(queues, wait, events)
    return fn(e0, e1, e2, d0, d1, alpha, _ptr(A), offA, lda, _ptr(B), offB, ldb, beta, _ptr(C), offC, ldc, nq, q, nw, w, e)


def clblasSsyr2k(order, uplo, transAB, N, K, alpha, A, offA, lda, B, offB, ldb, beta, C, offC, ldc,
                 queues=None, wait=None, events=None) -> int:
    """C <- alpha*op(A)*op(B)^T + alpha*op(B)*op(A)^T + beta*C on one triangle of C (src/clBLAS.h:8568-8589)."""
    return _abc(lib.clblasSsyr2k, order, uplo, transAB, N, K, alpha, A, offA, lda, B, offB, ldb, beta, C, offC, ldc,
                queues, wait, events)


def clblasDsyr2k(order, uplo, transAB, N, K, alpha, A, offA, lda, B, offB, ldb, beta, C, offC, ldc,
                 queues=None, wait=None, events=None) -> int:
    return _abc(lib.clblasDsyr2k, order, uplo, transAB, N, K, alpha, A, offA, lda, B, offB, ldb, beta, C, offC, ldc,
                queues, wait, events)


def clblasSsymm(order, side, uplo, M, N, alpha, A, offA, lda, B, offB, ldb, beta, C, offC, ldc,
                queues=None, wait=None, events=None) -> int:
    """C <- alpha*A*B + beta*C (Left) / alpha*B*A + beta*C (Right), A symmetric (src/clBLAS.h:8898-8919)."""
    return _abc(lib.clblasSsymm, order, side, uplo, M, N, alpha, A, offA, lda, B, offB, ldb, beta, C, offC, ldc,
                queues, wait, events)


def clblasDsymm(order, side, uplo, M, N, alpha, A, offA, lda, B, offB, ldb, beta, C, offC, ldc,
                queues=None, wait=None, events=None) -> int:
    return _abc(lib.clblasDsymm, order, side, uplo, M, N, alpha, A, offA, lda, B, offB, ldb, beta, C, offC, ldc,
                queues, wait, events)


def _cplx(ct, v):
    v = complex(v)
    return ct(v.real, v.imag)


def clblasCgemm(order, transA, transB, M, N, K, alpha, A, offA, lda, B, offB, ldb, beta, C, offC, ldc,
                queues=None, wait=None, events=None) -> int:
    """complex64 GEMM; alpha and beta are Python complex numbers (src/clBLAS.h:7538-7560)."""
    nq, q, nw, w, e = _queues_events(queues, wait, events)
    return lib.clblasCgemm(order, transA, transB, M, N, K, _cplx(FloatComplex, alpha), _ptr(A), offA, lda, _ptr(B), offB, ldb,
                           _cplx(FloatComplex, beta), _ptr(C), offC, ldc, nq, q, nw, w, e)


def clblasZgemm(order, transA, transB, M, N, K, alpha, A, offA, lda, B, offB, ldb, beta, C, offC, ldc,
                queues=None, wait=None, events=None) -> int:
    nq, q, nw, w, e = _queues_events(queues, wait, events)
    return lib.clblasZgemm(order, transA, transB, M, N, K, _cplx(DoubleComplex, alpha), _ptr(A), offA, lda, _ptr(B), offB, ldb,
                           _cplx(DoubleComplex, beta), _ptr(C), offC, ldc, nq, q, nw, w, e)


def clblasCtrsm(order, side, uplo, transA, diag, M, N, alpha, A, offA, lda, B, offB, ldb,
                queues=None, wait=None, events=None) -> int:
    """complex64 triangular solve, B overwritten by X; alpha is a Python complex number (src/clBLAS.h:8132-8151)."""
    nq, q, nw, w, e = _queues_events(queues, wait, events)
    return lib.clblasCtrsm(order, side, uplo, transA, diag, M, N, _cplx(FloatComplex, alpha), _ptr(A), offA, lda,
                           _ptr(B), offB, ldb, nq, q, nw, w, e)


def clblasZtrsm(order, side, uplo, transA, diag, M, N, alpha, A, offA, lda, B, offB, ldb,
                queues=None, wait=None, events=None) -> int:
    nq, q, nw, w, e = _queues_events(queues, wait, events)
    return lib.clblasZtrsm(order, side, uplo, transA, diag, M, N, _cplx(DoubleComplex, alpha), _ptr(A), offA, lda,
                           _ptr(B), offB, ldb, nq, q, nw, w, e)


# ---- matrix helpers (src/clBLAS.h:9665-10238).  Host matrices are numpy arrays, device matrices torch tensors or
# raw addresses; `queue` defaults to torch's current stream; the blocking variants are mirrored here, the Async
# ones are reachable through `lib`.
def _host_ptr(a):
    return a if a is None or isinstance(a, int) else a.ctypes.data


def _stream(queue):
    if queue is None:
        import torch
        queue = torch.cuda.current_stream()
    return _handle(queue)


def clblasMatrixSizeInfo(order, rows, columns, elemsize, padding):
    """(status, ld, fullsize in bytes) of a rows x columns matrix with `padding` extra elements per line."""
    ld, full = ctypes.c_size_t(), ctypes.c_size_t()
    st = lib.clblasMatrixSizeInfo(order, rows, columns, elemsize, padding, ctypes.byref(ld), ctypes.byref(full))
    return st, ld.value, full.value


def clblasWriteMatrix(order, sx, sy, element_size, A, offA, ldA, B, offB, ldB, queue=None) -> int:
    """Host matrix A (numpy) -> device matrix B, sx rows by sy columns."""
    return lib.clblasWriteMatrix(order, sx, sy, element_size, _host_ptr(A), offA, ldA, _ptr(B), offB, ldB, _stream(queue), 0, None)


def clblasReadMatrix(order, sx, sy, element_size, A, offA, ldA, B, offB, ldB, queue=None) -> int:
    """Device matrix A -> host matrix B (numpy)."""
    return lib.clblasReadMatrix(order, sx, sy, element_size, _ptr(A), offA, ldA, _host_ptr(B), offB, ldB, _stream(queue), 0, None)


def clblasCopyMatrix(order, sx, sy, element_size, A, offA, ldA, B, offB, ldB, queue=None) -> int:
    return lib.clblasCopyMatrix(order, sx, sy, element_size, _ptr(A), offA, ldA, _ptr(B), offB, ldB, _stream(queue), 0, None)


def clblasWriteSubMatrix(order, element_size, A, offA, ldA, nrA, ncA, xA, yA, B, offB, ldB, nrB, ncB, xB, yB, nx, ny, queue=None) -> int:
    return lib.clblasWriteSubMatrix(order, element_size, _host_ptr(A), offA, ldA, nrA, ncA, xA, yA, _ptr(B), offB, ldB, nrB, ncB,
                                    xB, yB, nx, ny, _stream(queue), 0, None)


def clblasReadSubMatrix(order, element_size, A, offA, ldA, nrA, ncA, xA, yA, B, offB, ldB, nrB, ncB, xB, yB, nx, ny, queue=None) -> int:
    return lib.clblasReadSubMatrix(order, element_size, _ptr(A), offA, ldA, nrA, ncA, xA, yA, _host_ptr(B), offB, ldB, nrB, ncB,
                                   xB, yB, nx, ny, _stream(queue), 0, None)


def clblasCopySubMatrix(order, element_size, A, offA, ldA, nrA, ncA, xA, yA, B, offB, ldB, nrB, ncB, xB, yB, nx, ny, queue=None) -> int:
    return lib.clblasCopySubMatrix(order, element_size, _ptr(A), offA, ldA, nrA, ncA, xA, yA, _ptr(B), offB, ldB, nrB, ncB,
                                   xB, yB, nx, ny, _stream(queue), 0, None)


def clblasFillVector(nb_elem, element_size, A, offA, pattern: bytes, queue=None) -> int:
    return lib.clblasFillVector(nb_elem, element_size, _ptr(A), offA, ctypes.c_char_p(pattern), _stream(queue), 0, None)


def clblasFillSubMatrix(order, element_size, A, offA, ldA, nrA, ncA, xA, yA, nx, ny, pattern: bytes, queue=None) -> int:
    return lib.clblasFillSubMatrix(order, element_size, _ptr(A), offA, ldA, nrA, ncA, xA, yA, nx, ny, ctypes.c_char_p(pattern),
                                   _stream(queue), 0, None)


def clblasFillMatrix(order, element_size, A, offA, ldA, nrA, ncA, pattern: bytes, queue=None) -> int:
    return lib.clblasFillMatrix(order, element_size, _ptr(A), offA, ldA, nrA, ncA, ctypes.c_char_p(pattern), _stream(queue), 0, None)


def clblasCtrmm(order, side, uplo, transA, diag, M, N, alpha, A, offA, lda, B, offB, ldb,
                queues=None, wait=None, events=None) -> int:
    """complex64 triangular product, B overwritten; alpha is a Python complex number (src/clBLAS.h:7839)."""
    nq, q, nw, w, e = _queues_events(queues, wait, events)
    return lib.clblasCtrmm(order, side, uplo, transA, diag, M, N, _cplx(FloatComplex, alpha), _ptr(A), offA, lda,
                           _ptr(B), offB, ldb, nq, q, nw, w, e)


def clblasZtrmm(order, side, uplo, transA, diag, M, N, alpha, A, offA, lda, B, offB, ldb,
                queues=None, wait=None, events=None) -> int:
    nq, q, nw, w, e = _queues_events(queues, wait, events)
    return lib.clblasZtrmm(order, side, uplo, transA, diag, M, N, _cplx(DoubleComplex, alpha), _ptr(A), offA, lda,
                           _ptr(B), offB, ldb, nq, q, nw, w, e)


def _complex_routine(name: str):
    """Builds the Python mirror of one complex symmetric / Hermitian routine (src/clBLAS.h:8417-9640): complex scalars
    are Python complex numbers, real ones (HERK's alpha and beta, HER2K's beta) floats."""
    prec = name[6]
    ct = FloatComplex if prec == "C" else DoubleComplex
    kind = name[7:]
    fn = getattr(lib, name)

    def conv(v, is_complex):
        return _cplx(ct, v) if is_complex else float(v)

    if kind in ("syrk", "herk"):
        def f(order, uplo, trans, N, K, alpha, A, offA, lda, beta, C, offC, ldc, queues=None, wait=None, events=None) -> int:
            nq, q, nw, w, e = _queues_events(queues, wait, events)
            cz = kind == "syrk"
            return fn(order, uplo, trans, N, K, conv(alpha, cz), _ptr(A), offA, lda, conv(beta, cz), _ptr(C), offC, ldc, nq, q, nw, w, e)
    elif kind in ("syr2k", "her2k"):
        def f(order, uplo, trans, N, K, alpha, A, offA, lda, B, offB, ldb, beta, C, offC, ldc, queues=None, wait=None, events=None) -> int:
            nq, q, nw, w, e = _queues_events(queues, wait, events)
            return fn(order, uplo, trans, N, K, conv(alpha, True), _ptr(A), offA, lda, _ptr(B), offB, ldb,
                      conv(beta, kind == "syr2k"), _ptr(C), offC, ldc, nq, q, nw, w, e)
    else:
        def f(order, side, uplo, M, N, alpha, A, offA, lda, B, offB, ldb, beta, C, offC, ldc, queues=None, wait=None, events=None) -> int:
            nq, q, nw, w, e = _queues_events(queues, wait, events)
            return fn(order, side, uplo, M, N, conv(alpha, True), _ptr(A), offA, lda, _ptr(B), offB, ldb, conv(beta, True),
                      _ptr(C), offC, ldc, nq, q, nw, w, e)
    f.__name__ = name
    return f


for _n in COMPLEX_SYM:
    globals()[_n] = _complex_routine(_n)


def _noalloc_limits():
    a, b = ctypes.c_size_t(), ctypes.c_size_t()
    lib.clblasB200NoAllocLimits(ctypes.byref(a), ctypes.byref(b))
    return a.value, b.value


NOALLOC_MAX_ORDER, NOALLOC_MAX_OTHER = _noalloc_limits()      # as compiled into the library


def clblasB200DtrsmNoAlloc(order, side, uplo, transA, diag, M, N, alpha, A, offA, lda, B, offB, ldb,
                           queues=None, wait=None, events=None) -> int:
    """clblasDtrsm for callers that may not allocate device memory while running (a process whose
    GPU memory all belongs to its own pool, a fixed-budget loop): the solve's workspace is a 12 MiB
    array resident in the library, so no allocation happens.  Order of A <= 4096, other dimension of
    B <= 8192, else clblasOutOfResources.  Calls that can overlap on the GPU share that array and race."""
    return _trsm(lib.clblasB200DtrsmNoAlloc, order, side, uplo, transA, diag, M, N, alpha, A, offA, lda, B, offB, ldb,
                 queues, wait, events)


def plan_shards(total: int, parts: int, align: int = 128):
    """Column-block boundaries for `parts` devices (clblasB200PlanShards)."""
    out = (ctypes.c_size_t * (parts + 1))()
    check(lib.clblasB200PlanShards(total, parts, align, out), "clblasB200PlanShards")
    return list(out)


def launch_count() -> int:
    return int(lib.clblasB200LaunchCount())


def probe_peak(kind: str, seconds: float = 0.2) -> float:
    """Measured issue-rate peak in TFLOP/s: kind "fp32" (FFMA) or "fp64" (FP64 tensor-core MMA)."""
    return float(lib.clblasB200ProbePeak(0 if kind == "fp32" else 1, seconds))


def device_fault() -> int:
    """Synchronises and returns the sticky bounded-wait failure flags (0 = healthy)."""
    return int(lib.clblasB200DeviceFault())


def last_gemm_kernel() -> str:
    return lib.clblasB200LastGemmKernel().decode()


def set_gemm_path(path: int) -> int:
    return lib.clblasB200SetGemmPath(path)


def last_gemm_variant() -> str:
    """Instantiation and mode of the kernel the calling thread's last GEMM ran (clblasB200LastGemmVariant)."""
    return lib.clblasB200LastGemmVariant().decode()


def workspace_alloc_count() -> int:
    """Workspace allocations made by the level-3 routines so far (clblasB200WorkspaceAllocCount)."""
    return int(lib.clblasB200WorkspaceAllocCount())


def panel_plan(columns: int, min_columns: int = 128, max_panels: int = 12):
    """Boundaries of the broadcast panels the sharded calls use (clblasB200PanelPlan)."""
    out = (ctypes.c_size_t * (max_panels + 1))()
    n = ctypes.c_uint()
    check(lib.clblasB200PanelPlan(columns, min_columns, max_panels, out, ctypes.byref(n)), "clblasB200PanelPlan")
    return list(out)[: n.value + 1]


# ---- one process per GPU: communicator and sharded forms -------------------------------------------------
UNIQUE_ID_BYTES = 128


def comm_get_unique_id() -> bytes:
    """128 bytes that identify a communicator about to be created; one rank makes them, all ranks use them."""
    buf = ctypes.create_string_buffer(UNIQUE_ID_BYTES)
    check(lib.clblasB200CommGetUniqueId(buf), "clblasB200CommGetUniqueId")
    return buf.raw


def comm_init_rank(unique_id: Optional[bytes], nranks: int, rank: int) -> int:
    """Joins the communicator (collective; the rank's device must be current).  Returns the handle."""
    h = ctypes.c_void_p()
    buf = ctypes.create_string_buffer(unique_id, UNIQUE_ID_BYTES) if unique_id is not None else None
    check(lib.clblasB200CommInitRank(ctypes.byref(h), buf, nranks, rank), "clblasB200CommInitRank")
    return h.value


def comm_destroy(comm) -> None:
    lib.clblasB200CommDestroy(comm)


def comm_from_process_group(group=None) -> int:
    """A communicator with one rank per rank of a torch.distributed process group: rank 0 draws the id, the
    group carries it to the others (the only use made of the group)."""
    import torch.distributed as dist
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    if world == 1:
        return comm_init_rank(None, 1, 0)
    box = [comm_get_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(box, src=dist.get_global_rank(group, 0) if group is not None else 0, group=group)
    return comm_init_rank(box[0], world, rank)


def _gemm_sharded(fn, order, transA, transB, M, N, K, alpha, A, offA, lda, B, offB, ldb, beta, C, offC, ldc, comm, root,
                  queues, wait, events):
    nq, q, nw, w, e = _queues_events(queues, wait, events)
    return fn(order, transA, transB, M, N, K, alpha, _ptr(A), offA, lda, _ptr(B), offB, ldb, beta, _ptr(C), offC, ldc,
              comm, root, nq, q, nw, w, e)


def clblasB200SgemmSharded(order, transA, transB, M, N, K, alpha, A, offA, lda, B, offB, ldb, beta, C, offC, ldc,
                           comm, root=0, queues=None, wait=None, events=None) -> int:
    """clblasSgemm on this rank's column block of op(B) and C (column-major; row-major: row block of op(A) and C);
    the other operand is broadcast from `root` in panels while the panel products run."""
    return _gemm_sharded(lib.clblasB200SgemmSharded, order, transA, transB, M, N, K, alpha, A, offA, lda, B, offB, ldb,
                         beta, C, offC, ldc, comm, root, queues, wait, events)


def clblasB200DgemmSharded(order, transA, transB, M, N, K, alpha, A, offA, lda, B, offB, ldb, beta, C, offC, ldc,
                           comm, root=0, queues=None, wait=None, events=None) -> int:
    return _gemm_sharded(lib.clblasB200DgemmSharded, order, transA, transB, M, N, K, alpha, A, offA, lda, B, offB, ldb,
                         beta, C, offC, ldc, comm, root, queues, wait, events)


def _trsm_sharded(fn, order, side, uplo, transA, diag, M, N, alpha, A, offA, lda, B, offB, ldb, comm, root, queues, wait, events):
    nq, q, nw, w, e = _queues_events(queues, wait, events)
    return fn(order, side, uplo, transA, diag, M, N, alpha, _ptr(A), offA, lda, _ptr(B), offB, ldb, comm, root, nq, q, nw, w, e)


def clblasB200StrsmSharded(order, side, uplo, transA, diag, M, N, alpha, A, offA, lda, B, offB, ldb, comm, root=0,
                           queues=None, wait=None, events=None) -> int:
    """clblasStrsm on this rank's block of right-hand sides; A is broadcast from `root` in panels the solve waits for."""
    return _trsm_sharded(lib.clblasB200StrsmSharded, order, side, uplo, transA, diag, M, N, alpha, A, offA, lda, B, offB, ldb,
                         comm, root, queues, wait, events)


def clblasB200DtrsmSharded(order, side, uplo, transA, diag, M, N, alpha, A, offA, lda, B, offB, ldb, comm, root=0,
                           queues=None, wait=None, events=None) -> int:
    return _trsm_sharded(lib.clblasB200DtrsmSharded, order, side, uplo, transA, diag, M, N, alpha, A, offA, lda, B, offB, ldb,
                         comm, root, queues, wait, events)
