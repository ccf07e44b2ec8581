"""Seeded TRMM cases (B <- alpha*op(A)*B or alpha*B*op(A)) shared by the oracle tests, the golden-vector
generator and the GPU parity tests; same conventions as tests/cases.py.  The triangular A carries NaN
outside the referenced triangle and on a unit diagonal, as the reference's generators do for the
triangular routines (src/tests/include/blas-random.h:260-263, :312-317)."""
from __future__ import annotations

import itertools

import numpy as np

import oracle
from oracle import ColumnMajor, Left, Lower, NonUnit, NoTrans, Right, RowMajor, Trans, ConjTrans, Unit, Upper
from tests.cases import DT, ORDERS, _min_ld


def trmm_case(prec, order, side, uplo, transA, diag, M, N, alpha=1.0, pad=(0, 0), off=(0, 0), mode="int", seed=12345):
    n = M if side == Left else N
    return dict(kind="trmm", prec=prec, order=order, side=side, uplo=uplo, transA=transA, diag=diag, M=M, N=N,
                alpha=alpha, lda=n + pad[0], ldb=_min_ld(order, NoTrans, M, N) + pad[1], offA=off[0], offB=off[1],
                mode=mode, seed=seed)


def trmm_logical(c):
    """Stored triangular A (n x n; NaN where it must not be read) and B (M x N)."""
    n = c["M"] if c["side"] == Left else c["N"]
    dt = DT[c["prec"]]
    g = oracle.rng(c["seed"], 17)
    if c["mode"] == "int":
        A = g.integers(-8, 9, size=(n, n)).astype(dt)
        B = g.integers(-8, 9, size=(c["M"], c["N"])).astype(dt)
    else:
        A = g.uniform(-1, 1, size=(n, n)).astype(dt)
        B = g.uniform(-1, 1, size=(c["M"], c["N"])).astype(dt)
    mask = np.triu(np.ones((n, n), dtype=bool), 1) if c["uplo"] == Lower else np.tril(np.ones((n, n), dtype=bool), -1)
    A[mask] = np.nan
    if c["diag"] == Unit:
        A[np.arange(n), np.arange(n)] = np.nan
    return A, B


def trmm_buffers(c, logical=None, tail=3):
    A, B = logical if logical is not None else trmm_logical(c)
    return (oracle.pack(A, c["order"], NoTrans, c["lda"], c["offA"], tail=tail),
            oracle.pack(B, c["order"], NoTrans, c["ldb"], c["offB"], tail=tail))


def trmm_exact(c, A, B):
    """alpha*op(T)*B or alpha*B*op(T) in float64 with T the clean triangle."""
    T = oracle.clean_triangle(A, c["uplo"], c["diag"]).astype(np.float64)
    T = T if c["transA"] == NoTrans else T.T
    B64 = B.astype(np.float64)
    return c["alpha"] * (T @ B64 if c["side"] == Left else B64 @ T), T


def golden_trmm_cases():
    out = {}
    k = 0
    for prec in "sd":
        for order, side, uplo, ta, diag in itertools.product(ORDERS, (Left, Right), (Upper, Lower), (NoTrans, Trans), (Unit, NonUnit)):
            M, N = [(9, 5), (16, 17), (7, 12)][k % 3]
            out[f"trmm_{prec}_{order}{side}{uplo}{ta}{diag}"] = trmm_case(
                prec, order, side, uplo, ta, diag, M, N, alpha=[1.0, -2.0, 0.5][k % 3], pad=(2, 3), off=(1, 4),
                mode=["int", "uniform"][k % 2], seed=400 + k)
            k += 1
    return out


def sweep_trmm_cases(prec, mode):
    cases = []
    seed = 7000
    for order, side, uplo, ta, diag in itertools.product(ORDERS, (Left, Right), (Upper, Lower), (NoTrans, Trans, ConjTrans), (Unit, NonUnit)):
        for (M, N) in ((8, 8), (17, 33), (128, 64), (130, 257), (300, 129)):
            seed += 1
            cases.append(trmm_case(prec, order, side, uplo, ta, diag, M, N, alpha=[1.0, 2.0, -3.0][seed % 3],
                                   pad=(seed % 5, seed % 7), off=(seed % 3, seed % 11), mode=mode, seed=seed))
    return cases
