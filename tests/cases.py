"""Seeded test cases shared by the oracle tests, the golden-vector generator and the GPU parity
tests.  Shapes follow the reference's correctness suite (src/tests/correctness/test-correctness.cpp:
SmallRange {8,16,17,32,62,64,128,144,256} :157-159, tiny shapes 1x1x1 / 2x1x3 / 3x2x1 / 4x3x2 /
17x13x1, leading dimensions and offsets of 500-502 elements :593-743 and :910-1070); the seed is
the suite's default 12345 (src/tests/include/BlasBase.h:44)."""
from __future__ import annotations

import itertools

import numpy as np

import oracle
from oracle import (ColumnMajor, Left, Lower, NonUnit, NoTrans, Right, RowMajor, Trans, ConjTrans, Unit, Upper)

ORDERS = (ColumnMajor, RowMajor)
TRANS = (NoTrans, Trans, ConjTrans)
DT = {"s": np.float32, "d": np.float64}


def _min_ld(order, trans, rows, cols):
    inner, _ = oracle.stored_shape(order, trans, rows, cols)
    return max(inner, 1)


def gemm_case(prec, order, transA, transB, M, N, K, alpha=1.5, beta=0.5, pad=(0, 0, 0), off=(0, 0, 0),
              mode="uniform", seed=12345):
    """pad = extra leading dimension beyond the minimum for A, B, C; off = element offsets."""
    return dict(kind="gemm", prec=prec, order=order, transA=transA, transB=transB, M=M, N=N, K=K,
                alpha=alpha, beta=beta,
                lda=_min_ld(order, transA, M, K) + pad[0], ldb=_min_ld(order, transB, K, N) + pad[1],
                ldc=_min_ld(order, NoTrans, M, N) + pad[2], offA=off[0], offB=off[1], offC=off[2],
                mode=mode, seed=seed)


def gemm_logical(c):
    """Logical op(A) (MxK), op(B) (KxN), C (MxN) of a case, from its seed."""
    dt = DT[c["prec"]]
    M, N, K = c["M"], c["N"], c["K"]
    if c["mode"] == "int":
        return oracle.exact_int_gemm_inputs(M, N, K, c["alpha"], c["beta"], dt, c["seed"])
    if c["mode"] == "normal":
        return (oracle.normal((M, K), dt, c["seed"], 1), oracle.normal((K, N), dt, c["seed"], 2),
                oracle.normal((M, N), dt, c["seed"], 3))
    return (oracle.uniform((M, K), dt, c["seed"], 1), oracle.uniform((K, N), dt, c["seed"], 2),
            oracle.uniform((M, N), dt, c["seed"], 3))


def gemm_buffers(c, logical=None, tail=3):
    """Flat A, B, C buffers (NaN in every element that is not part of a matrix)."""
    opA, opB, C = logical if logical is not None else gemm_logical(c)
    A = oracle.pack(opA, c["order"], c["transA"], c["lda"], c["offA"], tail=tail)
    B = oracle.pack(opB, c["order"], c["transB"], c["ldb"], c["offB"], tail=tail)
    Cb = oracle.pack(C, c["order"], NoTrans, c["ldc"], c["offC"], tail=tail)
    return A, B, Cb


def trsm_case(prec, order, side, uplo, transA, diag, M, N, alpha=1.0, pad=(0, 0), off=(0, 0), seed=12345):
    n = M if side == Left else N
    return dict(kind="trsm", prec=prec, order=order, side=side, uplo=uplo, transA=transA, diag=diag, M=M, N=N,
                alpha=alpha, lda=n + pad[0], ldb=_min_ld(order, NoTrans, M, N) + pad[1], offA=off[0], offB=off[1],
                seed=seed)


def trsm_logical(c):
    """Stored triangular A (n x n, NaN outside the referenced triangle) and B (M x N)."""
    n = c["M"] if c["side"] == Left else c["N"]
    return oracle.trsm_inputs(n, (c["M"], c["N"]), c["uplo"], c["diag"], DT[c["prec"]], c["seed"])


def trsm_buffers(c, logical=None, tail=3):
    A, B = logical if logical is not None else trsm_logical(c)
    Ab = oracle.pack(A, c["order"], NoTrans, c["lda"], c["offA"], tail=tail)
    Bb = oracle.pack(B, c["order"], NoTrans, c["ldb"], c["offB"], tail=tail)
    return Ab, Bb


def trsm_op_triangle(c, A):
    """Dense op(A) with zeros outside the triangle and ones on a unit diagonal."""
    T = oracle.clean_triangle(A, c["uplo"], c["diag"])
    return T if c["transA"] == NoTrans else T.T


# ---- case sets ---------------------------------------------------------------------------------

SMALL_RANGE = (8, 16, 17, 32, 62, 64, 128, 144, 256)
TINY = ((1, 1, 1), (2, 1, 3), (3, 2, 1), (4, 3, 2), (17, 13, 1))


def golden_gemm_cases():
    """Small cases whose reference outputs are committed under tests/golden/."""
    out = {}
    k = 0
    for prec in "sd":
        for order, ta, tb in itertools.product(ORDERS, (NoTrans, Trans), (NoTrans, Trans)):
            M, N, K = [(17, 13, 9), (32, 8, 33), (5, 62, 16), (64, 17, 8)][k % 4]
            out[f"gemm_{prec}_{order}{ta}{tb}_int"] = gemm_case(prec, order, ta, tb, M, N, K, alpha=2.0, beta=3.0,
                                                                 pad=(3, 1, 2), off=(5, 2, 7), mode="int", seed=100 + k)
            out[f"gemm_{prec}_{order}{ta}{tb}_uni"] = gemm_case(prec, order, ta, tb, N, M, K + 1, alpha=1.5, beta=0.5,
                                                                 pad=(0, 2, 1), off=(0, 1, 0), mode="uniform", seed=200 + k)
            k += 1
    return out


def golden_trsm_cases():
    out = {}
    k = 0
    for prec in "sd":
        for order, side, uplo, ta, diag in itertools.product(ORDERS, (Left, Right), (Upper, Lower), (NoTrans, Trans),
                                                             (Unit, NonUnit)):
            M, N = [(9, 5), (16, 17), (7, 12)][k % 3]
            out[f"trsm_{prec}_{order}{side}{uplo}{ta}{diag}"] = trsm_case(prec, order, side, uplo, ta, diag, M, N,
                                                                          alpha=[1.0, -2.0, 0.5][k % 3], pad=(2, 3),
                                                                          off=(1, 4), seed=300 + k)
            k += 1
    return out


def sweep_gemm_cases(prec, mode):
    """The GPU parity sweep: reference-style size matrix, both orders, all transposes."""
    cases = []
    seed = 1000
    for order in ORDERS:
        for ta, tb in itertools.product(TRANS, TRANS):
            for (M, N, K) in ((8, 8, 8), (17, 17, 17), (62, 64, 32), (64, 62, 144), (128, 144, 17), (256, 128, 62),
                              (129, 257, 65)):
                seed += 1
                cases.append(gemm_case(prec, order, ta, tb, M, N, K, alpha=2.0 if mode == "int" else 1.5,
                                       beta=3.0 if mode == "int" else 0.5, mode=mode, seed=seed))
            for (M, N, K) in TINY:
                seed += 1
                cases.append(gemm_case(prec, order, ta, tb, M, N, K, alpha=1.0, beta=1.0, mode=mode, seed=seed))
        # big leading dimensions and offsets (test-correctness.cpp "BigLDA" 500/501/502 and offsets)
        for ta, tb in itertools.product((NoTrans, Trans), (NoTrans, Trans)):
            seed += 1
            cases.append(gemm_case(prec, order, ta, tb, 63, 64, 65, alpha=2.0, beta=1.0, pad=(437, 436, 439),
                                   off=(500, 501, 502), mode=mode, seed=seed))
            seed += 1
            cases.append(gemm_case(prec, order, ta, tb, 200, 130, 77, alpha=-1.0, beta=0.0, pad=(1, 3, 5),
                                   off=(1, 2, 3), mode=mode, seed=seed))
    return cases


def sweep_trsm_cases(prec):
    cases = []
    seed = 5000
    for order, side, uplo, ta, diag in itertools.product(ORDERS, (Left, Right), (Upper, Lower), TRANS, (Unit, NonUnit)):
        for (M, N) in ((8, 8), (17, 33), (128, 64), (130, 257), (300, 129)):
            seed += 1
            cases.append(trsm_case(prec, order, side, uplo, ta, diag, M, N, alpha=[1.0, 2.5, -0.5][seed % 3],
                                   pad=(seed % 5, seed % 7), off=(seed % 3, seed % 11), seed=seed))
    return cases
