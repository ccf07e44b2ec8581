"""CPU oracle for the level-3 hot path -- TEST INFRASTRUCTURE ONLY.

Only ``tests/``, ``__graft_entry__.smoke()`` and the CPU-baseline legs of ``bench.py`` may import
this package; the product (``clblas_b200``) never does.

Two checkers live here:

* ``impl="port"``: ``oracle_blas.c``, a plain-C restatement of the reference's own CPU BLAS
  (``NaiveBlas::gemm`` / ``NaiveBlas::trsm``, src/library/tools/ktest/naive/naive_blas.cpp:546-578,
  :632-690);
* ``impl="ref"``: that reference file itself, compiled from the reference tree into
  ``oracle/_ref/libnaive_ref.so`` by ``oracle/Makefile`` (available wherever it was built).

Both take flat buffers with element offsets and leading dimensions, like the clBLAS entry points.
The module also holds the seeded input generators (the reference tests' exact-integer GEMM inputs,
src/tests/include/blas-random.h:29-94, and diagonally dominant triangular systems with NaN outside
the referenced triangle, :175-342) and the tolerance formulas the parity tests use.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))

RowMajor, ColumnMajor = 0, 1
NoTrans, Trans, ConjTrans = 0, 1, 2
Upper, Lower = 0, 1
Unit, NonUnit = 0, 1
Left, Right = 0, 1

_U = {np.dtype(np.float32): 2.0 ** -24, np.dtype(np.float64): 2.0 ** -53}


def unit_roundoff(dtype) -> float:
    return _U[np.dtype(dtype)]


def build(force: bool = False) -> None:
    """Compile the C restatement and, where the reference tree exists, the reference's own file."""
    port = os.path.join(_HERE, "liboracle_blas.so")
    src = os.path.join(_HERE, "oracle_blas.c")
    ref = os.path.join(_HERE, "_ref", "libnaive_ref.so")
    stale = (not os.path.exists(port)) or os.path.getmtime(port) < os.path.getmtime(src)
    # the reference tree: REF_ROOT, or a checkout named "reference" beside this repository
    ref_root = os.environ.get("REF_ROOT") or os.path.normpath(os.path.join(_HERE, "..", "..", "reference"))
    ref_possible = os.path.exists(os.path.join(ref_root, "src", "library", "tools", "ktest", "naive", "naive_blas.cpp"))
    shim = os.path.join(_HERE, "ref_shim.cpp")
    if ref_possible and os.path.exists(ref) and os.path.getmtime(ref) < os.path.getmtime(shim):
        force = True
    if force or stale or (ref_possible and not os.path.exists(ref)):
        subprocess.run(["make", "-C", _HERE, "-B" if force else "-s", f"REF_ROOT={ref_root}"], check=True,
                       stdout=subprocess.DEVNULL)


_libs: dict[str, ctypes.CDLL] = {}


def _lib(impl: str) -> ctypes.CDLL:
    if impl in _libs:
        return _libs[impl]
    if impl == "port":
        path, prefix = os.path.join(_HERE, "liboracle_blas.so"), "oracle_"
        if not os.path.exists(path):
            build()
    elif impl == "ref":
        path, prefix = os.path.join(_HERE, "_ref", "libnaive_ref.so"), "ref_"
    else:
        raise ValueError(impl)
    lib = ctypes.CDLL(path)
    sz, i = ctypes.c_size_t, ctypes.c_int
    for p, ct in (("s", ctypes.c_float), ("d", ctypes.c_double)):
        ptr = ctypes.c_void_p
        getattr(lib, f"{prefix}{p}gemm").argtypes = [i, i, i, sz, sz, sz, ct, ptr, sz, ptr, sz, ct, ptr, sz]
        getattr(lib, f"{prefix}{p}gemm").restype = None
        getattr(lib, f"{prefix}{p}trsm").argtypes = [i, i, i, i, i, sz, sz, ct, ptr, sz, ptr, sz]
        getattr(lib, f"{prefix}{p}trsm").restype = None
        getattr(lib, f"{prefix}{p}trmm").argtypes = [i, i, i, i, i, sz, sz, ct, ptr, sz, ptr, sz]
        getattr(lib, f"{prefix}{p}trmm").restype = None
        getattr(lib, f"{prefix}{p}syrk").argtypes = [i, i, i, sz, sz, ct, ptr, sz, ct, ptr, sz]
        getattr(lib, f"{prefix}{p}syrk").restype = None
        getattr(lib, f"{prefix}{p}syr2k").argtypes = [i, i, i, sz, sz, ct, ptr, sz, ptr, sz, ct, ptr, sz]
        getattr(lib, f"{prefix}{p}syr2k").restype = None
        if prefix == "oracle_":      # the reference's naive BLAS has no symm
            getattr(lib, f"{prefix}{p}symm").argtypes = [i, i, i, sz, sz, ct, ptr, sz, ptr, sz, ct, ptr, sz]
            getattr(lib, f"{prefix}{p}symm").restype = None
    for p, ct in (("c", ctypes.c_float), ("z", ctypes.c_double)):
        ptr = ctypes.c_void_p
        getattr(lib, f"{prefix}{p}gemm").argtypes = [i, i, i, sz, sz, sz, ct, ct, ptr, sz, ptr, sz, ct, ct, ptr, sz]
        getattr(lib, f"{prefix}{p}gemm").restype = None
        getattr(lib, f"{prefix}{p}trsm").argtypes = [i, i, i, i, i, sz, sz, ct, ct, ptr, sz, ptr, sz]
        getattr(lib, f"{prefix}{p}trsm").restype = None
        getattr(lib, f"{prefix}{p}trmm").argtypes = [i, i, i, i, i, sz, sz, ct, ct, ptr, sz, ptr, sz]
        getattr(lib, f"{prefix}{p}trmm").restype = None
        if prefix == "oracle_":      # herm flag after trans / uplo; the reference's naive BLAS has only the symmetric updates
            getattr(lib, f"{prefix}{p}syrk").argtypes = [i, i, i, i, sz, sz, ct, ct, ptr, sz, ct, ct, ptr, sz]
            getattr(lib, f"{prefix}{p}syr2k").argtypes = [i, i, i, i, sz, sz, ct, ct, ptr, sz, ptr, sz, ct, ct, ptr, sz]
            getattr(lib, f"{prefix}{p}symm").argtypes = [i, i, i, i, sz, sz, ct, ct, ptr, sz, ptr, sz, ct, ct, ptr, sz]
            getattr(lib, f"{prefix}{p}symm").restype = None
        else:
            getattr(lib, f"{prefix}{p}syrk").argtypes = [i, i, i, sz, sz, ct, ct, ptr, sz, ct, ct, ptr, sz]
            getattr(lib, f"{prefix}{p}syr2k").argtypes = [i, i, i, sz, sz, ct, ct, ptr, sz, ptr, sz, ct, ct, ptr, sz]
        getattr(lib, f"{prefix}{p}syrk").restype = None
        getattr(lib, f"{prefix}{p}syr2k").restype = None
    lib._prefix = prefix
    _libs[impl] = lib
    return lib


def have_ref() -> bool:
    return os.path.exists(os.path.join(_HERE, "_ref", "libnaive_ref.so"))


def _p(arr: np.ndarray, off: int) -> ctypes.c_void_p:
    assert arr.flags["C_CONTIGUOUS"] and arr.ndim == 1
    return ctypes.c_void_p(arr.ctypes.data + off * arr.itemsize)


def gemm(order, transA, transB, M, N, K, alpha, A, offA, lda, B, offB, ldb, beta, C, offC, ldc,
         impl: str = "port") -> None:
    """C <- alpha*op(A)*op(B) + beta*C in place on the flat buffer C (same dtype for all three)."""
    lib = _lib(impl)
    p = "s" if C.dtype == np.float32 else "d"
    fn = getattr(lib, f"{lib._prefix}{p}gemm")
    fn(order, transA, transB, M, N, K, alpha, _p(A, offA), lda, _p(B, offB), ldb, beta, _p(C, offC), ldc)


def trsm(order, side, uplo, transA, diag, M, N, alpha, A, offA, lda, B, offB, ldb,
         impl: str = "port") -> None:
    """Solve op(A) X = alpha B (Left) / X op(A) = alpha B (Right) in place on the flat buffer B."""
    lib = _lib(impl)
    p = "s" if B.dtype == np.float32 else "d"
    fn = getattr(lib, f"{lib._prefix}{p}trsm")
    fn(order, side, uplo, transA, diag, M, N, alpha, _p(A, offA), lda, _p(B, offB), ldb)


def trmm(order, side, uplo, transA, diag, M, N, alpha, A, offA, lda, B, offB, ldb,
         impl: str = "port") -> None:
    """B <- alpha op(A) B (Left) / alpha B op(A) (Right) in place on the flat buffer B."""
    lib = _lib(impl)
    p = "s" if B.dtype == np.float32 else "d"
    fn = getattr(lib, f"{lib._prefix}{p}trmm")
    fn(order, side, uplo, transA, diag, M, N, alpha, _p(A, offA), lda, _p(B, offB), ldb)


def cgemm(order, transA, transB, M, N, K, alpha, A, offA, lda, B, offB, ldb, beta, C, offC, ldc, impl: str = "port") -> None:
    """Complex GEMM in place on the flat complex64 / complex128 buffer C; alpha, beta Python complex numbers."""
    lib = _lib(impl)
    p = "c" if C.dtype == np.complex64 else "z"
    alpha, beta = complex(alpha), complex(beta)
    fn = getattr(lib, f"{lib._prefix}{p}gemm")
    fn(order, transA, transB, M, N, K, alpha.real, alpha.imag, _p(A, offA), lda, _p(B, offB), ldb, beta.real, beta.imag,
       _p(C, offC), ldc)


def ctrsm(order, side, uplo, transA, diag, M, N, alpha, A, offA, lda, B, offB, ldb, impl: str = "port") -> None:
    """Complex triangular solve in place on the flat complex buffer B; alpha a Python complex number."""
    lib = _lib(impl)
    p = "c" if B.dtype == np.complex64 else "z"
    alpha = complex(alpha)
    fn = getattr(lib, f"{lib._prefix}{p}trsm")
    fn(order, side, uplo, transA, diag, M, N, alpha.real, alpha.imag, _p(A, offA), lda, _p(B, offB), ldb)


def ctrmm(order, side, uplo, transA, diag, M, N, alpha, A, offA, lda, B, offB, ldb, impl: str = "port") -> None:
    """Complex triangular product in place on the flat complex buffer B; alpha a Python complex number."""
    lib = _lib(impl)
    alpha = complex(alpha)
    fn = getattr(lib, f"{lib._prefix}{'c' if B.dtype == np.complex64 else 'z'}trmm")
    fn(order, side, uplo, transA, diag, M, N, alpha.real, alpha.imag, _p(A, offA), lda, _p(B, offB), ldb)


def _cz(arr):
    return "c" if arr.dtype == np.complex64 else "z"


def csyrk(order, uplo, trans, N, K, alpha, A, offA, lda, beta, C, offC, ldc, herm=False, impl: str = "port") -> None:
    """Complex SYRK (herm=False; impl "ref" = NaiveBlas::syrk) or HERK (herm=True, port only) in place on C."""
    lib = _lib(impl)
    alpha, beta = complex(alpha), complex(beta)
    fn = getattr(lib, f"{lib._prefix}{_cz(C)}syrk")
    if impl == "port":
        fn(order, uplo, trans, int(herm), N, K, alpha.real, alpha.imag, _p(A, offA), lda, beta.real, beta.imag, _p(C, offC), ldc)
    else:
        assert not herm
        fn(order, uplo, trans, N, K, alpha.real, alpha.imag, _p(A, offA), lda, beta.real, beta.imag, _p(C, offC), ldc)


def csyr2k(order, uplo, trans, N, K, alpha, A, offA, lda, B, offB, ldb, beta, C, offC, ldc, herm=False, impl: str = "port") -> None:
    """Complex SYR2K (herm=False; impl "ref" = NaiveBlas::syr2k) or HER2K (herm=True, port only) in place on C."""
    lib = _lib(impl)
    alpha, beta = complex(alpha), complex(beta)
    fn = getattr(lib, f"{lib._prefix}{_cz(C)}syr2k")
    if impl == "port":
        fn(order, uplo, trans, int(herm), N, K, alpha.real, alpha.imag, _p(A, offA), lda, _p(B, offB), ldb, beta.real, beta.imag,
           _p(C, offC), ldc)
    else:
        assert not herm
        fn(order, uplo, trans, N, K, alpha.real, alpha.imag, _p(A, offA), lda, _p(B, offB), ldb, beta.real, beta.imag, _p(C, offC), ldc)


def csymm(order, side, uplo, M, N, alpha, A, offA, lda, B, offB, ldb, beta, C, offC, ldc, herm=False) -> None:
    """Complex SYMM (herm=False) or HEMM (herm=True) in place on C; port only (Netlib definition)."""
    lib = _lib("port")
    alpha, beta = complex(alpha), complex(beta)
    fn = getattr(lib, f"oracle_{_cz(C)}symm")
    fn(order, side, uplo, int(herm), M, N, alpha.real, alpha.imag, _p(A, offA), lda, _p(B, offB), ldb, beta.real, beta.imag,
       _p(C, offC), ldc)


def syrk(order, uplo, trans, N, K, alpha, A, offA, lda, beta, C, offC, ldc, impl: str = "port") -> None:
    """C <- alpha op(A) op(A)^T + beta C on the uplo triangle, in place on the flat buffer C."""
    lib = _lib(impl)
    p = "s" if C.dtype == np.float32 else "d"
    fn = getattr(lib, f"{lib._prefix}{p}syrk")
    fn(order, uplo, trans, N, K, alpha, _p(A, offA), lda, beta, _p(C, offC), ldc)


def syr2k(order, uplo, trans, N, K, alpha, A, offA, lda, B, offB, ldb, beta, C, offC, ldc, impl: str = "port") -> None:
    """C <- alpha (op(A) op(B)^T + op(B) op(A)^T) + beta C on the uplo triangle, in place on the flat buffer C."""
    lib = _lib(impl)
    p = "s" if C.dtype == np.float32 else "d"
    fn = getattr(lib, f"{lib._prefix}{p}syr2k")
    fn(order, uplo, trans, N, K, alpha, _p(A, offA), lda, _p(B, offB), ldb, beta, _p(C, offC), ldc)


def symm(order, side, uplo, M, N, alpha, A, offA, lda, B, offB, ldb, beta, C, offC, ldc) -> None:
    """C <- alpha A B + beta C (Left) or alpha B A + beta C (Right), A symmetric with the uplo triangle stored.
    Port only: the reference's naive BLAS has no symm (its tests call an external Fortran BLAS)."""
    lib = _lib("port")
    p = "s" if C.dtype == np.float32 else "d"
    fn = getattr(lib, f"oracle_{p}symm")
    fn(order, side, uplo, M, N, alpha, _p(A, offA), lda, _p(B, offB), ldb, beta, _p(C, offC), ldc)


# --------------------------------------------------------------------------------------------
# flat-buffer helpers
# --------------------------------------------------------------------------------------------

def stored_shape(order, trans, rows, cols):
    """(contiguous extent, number of strides) of op(X) = rows x cols as stored in memory."""
    tra = (order == ColumnMajor and trans == NoTrans) or (order == RowMajor and trans != NoTrans)
    return (rows, cols) if tra else (cols, rows)


def buffer_len(order, trans, rows, cols, ld, off):
    inner, outer = stored_shape(order, trans, rows, cols)
    return off + (outer - 1) * ld + inner if inner and outer else off


def view(buf, order, trans, rows, cols, ld, off):
    """Strided numpy view of the logical rows x cols matrix op(X) living in the flat buffer."""
    tra = (order == ColumnMajor and trans == NoTrans) or (order == RowMajor and trans != NoTrans)
    it = buf.itemsize
    strides = (it, ld * it) if tra else (ld * it, it)
    return np.lib.stride_tricks.as_strided(buf[off:], shape=(rows, cols), strides=strides)


def pack(mat, order, trans, ld, off, pad_value=np.nan, tail=0):
    """Place logical matrix `mat` (= op(X)) into a fresh flat buffer; every element that does not
    belong to the matrix (the `off` leading elements, the ld padding, `tail` trailing elements)
    is `pad_value` so that illegal reads poison the result and illegal writes are detectable."""
    rows, cols = mat.shape
    n = buffer_len(order, trans, rows, cols, ld, off) + tail
    buf = np.full(n, pad_value, dtype=mat.dtype)
    if rows and cols:
        view(buf, order, trans, rows, cols, ld, off)[...] = mat
    return buf


def outside_mask(n, order, trans, rows, cols, ld, off):
    """Boolean mask over a flat buffer of length n: True where the element is NOT part of the matrix."""
    m = np.ones(n, dtype=bool)
    if rows and cols:
        view(m, order, trans, rows, cols, ld, off)[...] = False
    return m


# --------------------------------------------------------------------------------------------
# seeded inputs
# --------------------------------------------------------------------------------------------

def rng(seed=12345, stream=0):
    """Counter-based generator (Philox) keyed by (seed, stream); seed 12345 is the reference
    tests' default (src/tests/include/BlasBase.h:44)."""
    return np.random.Generator(np.random.Philox(key=[seed, stream]))


def uniform(shape, dtype, seed=12345, stream=0, lo=-1.0, hi=1.0):
    return rng(seed, stream).uniform(lo, hi, size=shape).astype(dtype)


def normal(shape, dtype, seed=12345, stream=0):
    return rng(seed, stream).standard_normal(size=shape).astype(dtype)


def exact_int_gemm_inputs(M, N, K, alpha, beta, dtype, seed=12345):
    """Integer-valued A, B, C in the style of randomGemmMatrices (blas-random.h:29-94): entries
    +-(r mod bound) with bound = sqrt((K-1)*U/(|alpha| K^2)) for A and B and sqrt(U/(|beta| K)) for C,
    U = 2^23 (fp32) or 2^52 (fp64) (test-limits.h:21-22).  With alpha and beta integer-valued every
    product and partial sum is exactly representable, so any summation order gives the same bits."""
    U = 2.0 ** 23 if np.dtype(dtype) == np.float32 else 2.0 ** 52
    g = rng(seed, 7)
    Kk = max(K, 1)
    bound_ab = int(np.sqrt(max(Kk - 1, 1) * U / (max(abs(alpha), 1.0) * Kk * Kk)))
    bound_ab = max(min(bound_ab, 1 << 20), 1)
    bound_c = int(np.sqrt(U / (max(abs(beta), 1.0) * Kk)))
    bound_c = max(min(bound_c, 1 << 20), 1)

    def draw(shape, bound):
        mag = g.integers(0, bound, size=shape, endpoint=False)
        sign = g.integers(0, 2, size=shape) * 2 - 1
        return (mag * sign).astype(dtype)

    return draw((M, K), bound_ab), draw((K, N), bound_ab), draw((M, N), bound_c)


def trsm_inputs(order_n, N_rhs_shape, uplo, diag, dtype, seed=12345, poison=True):
    """Triangular A (order_n x order_n, logical, op not applied) and right-hand side B in the style of
    randomTrsmMatrices (blas-random.h:175-342): diagonal magnitudes in [max/100, max] with max = 2^7
    (fp32) / 2^5 (fp64) (test-limits.h:24-27), off-diagonal entries small enough that every row stays
    diagonally dominant, NaN everywhere outside the referenced triangle and, for a unit diagonal, on
    the diagonal as well (blas-random.h:260-263, :312-317)."""
    g = rng(seed, 11)
    n = order_n
    amax = 2.0 ** 7 if np.dtype(dtype) == np.float32 else 2.0 ** 5
    A = g.uniform(-1.0, 1.0, size=(n, n))
    dsign = g.integers(0, 2, size=n) * 2 - 1
    dmag = g.uniform(amax / 100.0, amax, size=n)
    # scale off-diagonals so that sum_j |a_ij| <= |a_ii| / 2
    scale = (dmag / 2.0) / np.maximum(n - 1, 1)
    A = A * scale[:, None]
    tri = np.tril(A, -1) if uplo == Lower else np.triu(A, 1)
    if diag == NonUnit:
        tri = tri + np.diag(dsign * dmag)
    else:
        # keep a unit-diagonal system well conditioned: shrink off-diagonals below 1/n
        tri = tri / amax
    A = tri.astype(dtype)
    if poison:
        mask = np.triu(np.ones((n, n), dtype=bool), 1) if uplo == Lower else np.tril(np.ones((n, n), dtype=bool), -1)
        A[mask] = np.nan
        if diag == Unit:
            A[np.arange(n), np.arange(n)] = np.nan
    B = g.uniform(-8.0, 8.0, size=N_rhs_shape).astype(dtype)
    return A, B


def clean_triangle(A, uplo, diag):
    """The triangular matrix a TRSM actually uses: zeros outside the triangle, ones on a unit diagonal."""
    T = np.tril(np.nan_to_num(A, nan=0.0)) if uplo == Lower else np.triu(np.nan_to_num(A, nan=0.0))
    if diag == Unit:
        T = T.copy()
        T[np.arange(T.shape[0]), np.arange(T.shape[0])] = 1.0
    return T


# --------------------------------------------------------------------------------------------
# tolerances
# --------------------------------------------------------------------------------------------

def gemm_error_ratio(C_got, alpha, opA, opB, beta, C_in, K, dtype):
    """max_ij |C_got - C_exact| / (|alpha| (|A||B|)_ij + |beta| |C_in|_ij) divided by the allowed
    4*K*u, with C_exact and the denominator computed in float64 from the same inputs.  A value
    <= 1 passes the stated tolerance."""
    A64, B64 = opA.astype(np.float64), opB.astype(np.float64)
    exact = alpha * (A64 @ B64)
    denom = abs(alpha) * (np.abs(A64) @ np.abs(B64))
    if beta != 0:
        exact = exact + beta * C_in.astype(np.float64)
        denom = denom + abs(beta) * np.abs(C_in.astype(np.float64))
    denom = np.where(denom == 0, np.finfo(np.float64).tiny, denom)
    err = np.abs(C_got.astype(np.float64) - exact) / denom
    bound = 4.0 * max(K, 1) * unit_roundoff(dtype)
    return float(np.max(err) / bound) if err.size else 0.0


def trsm_backward_ratio(X, alpha, T, B_in, side, dtype):
    """max_ij |alpha B - op(T) X|_ij / (|op(T)||X| + |alpha||B|)_ij (Left; X op(T) for Right) divided
    by the allowed 4*M*u, M the order of the triangular matrix.  T is op(A) already applied, dense
    with zeros outside the triangle.  A value <= 1 passes."""
    T64, X64, B64 = T.astype(np.float64), X.astype(np.float64), B_in.astype(np.float64)
    if side == Left:
        res = alpha * B64 - T64 @ X64
        den = np.abs(T64) @ np.abs(X64) + abs(alpha) * np.abs(B64)
    else:
        res = alpha * B64 - X64 @ T64
        den = np.abs(X64) @ np.abs(T64) + abs(alpha) * np.abs(B64)
    den = np.where(den == 0, np.finfo(np.float64).tiny, den)
    bound = 4.0 * T.shape[0] * unit_roundoff(dtype)
    return float(np.max(np.abs(res) / den) / bound) if res.size else 0.0


def op(mat, trans):
    return mat if trans == NoTrans else mat.T


def trsm_delta(side, uplo, transA, diag, A, B, alpha, dtype):
    """The reference's element-wise acceptance bound for TRSM, trsmDelta
    (src/tests/correctness/trsm-delta.h:44-240), on logical matrices: A the stored triangular matrix
    (only its diagonal is read), B the right-hand sides BEFORE the solve.  Returns delta (M x N): the
    reference accepts a result when |X_blas - X_library| <= delta entry by entry
    (compareMatrices, src/tests/include/matrix.h:301-329).

    delta = (error of plain substitution) + (extra error of the reference's blocked algorithm):
    with e[i, k] = |B[i, k] / A[i, i]| * DELTA_0 * |alpha| (DELTA_0 = 2^-20 for float, 2^-50 for double; the
    division only for a non-unit diagonal), the first term is the running sum of e along the direction of
    substitution, the second one bsize (32) times a weighted sum of that running sum at the same offset inside
    each block of 32, the weights counting how many later blocks a block's error propagates into.
    The Right / lower-triangular branch of the reference stops its block loop at (k + 31) / 32, so it adds
    at most the term of k's own block; that is restated as it stands."""
    d0 = 2.0 ** -20 if np.dtype(dtype) == np.float32 else 2.0 ** -50
    bs = 32
    B64 = np.abs(np.asarray(B, dtype=np.float64))
    M, N = B64.shape
    is_upper = (uplo == Upper) == (transA == NoTrans)
    dd = np.abs(np.diagonal(np.asarray(A, dtype=np.float64))) if diag == NonUnit else None
    amod = abs(alpha)
    block = np.zeros((M, N))
    if side == Left:
        e = (B64 / dd[:, None] if dd is not None else B64) * d0 * amod
        gauss = np.cumsum(e[::-1], axis=0)[::-1] if is_upper else np.cumsum(e, axis=0)
        nblk = (M + bs - 1) // bs
        for i in range(M):
            if is_upper:
                js, zs = range(i // bs, nblk), range(1, nblk - i // bs + 1)
            else:
                js, zs = range(0, i // bs + 1), range(i // bs + 1, 0, -1)
            for j, z in zip(js, zs):
                idx = j * bs + i % bs
                if idx < M:
                    block[i] += z * gauss[idx]
    else:
        e = (B64 / dd[None, :] if dd is not None else B64) * d0 * amod
        gauss = np.cumsum(e, axis=1) if is_upper else np.cumsum(e[:, ::-1], axis=1)[:, ::-1]
        for k in range(N):
            if is_upper:
                js, zs = range(0, k // bs + 1), range(k // bs + 1, 0, -1)
            else:
                js, zs = range(k // bs, (k + bs - 1) // bs), range(1, bs + 2)
            for j, z in zip(js, zs):
                idx = j * bs + k % bs
                if idx < N:
                    block[:, k] += z * gauss[:, idx]
    return gauss + block * bs
