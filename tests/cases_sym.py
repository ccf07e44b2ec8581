"""Seeded SYR2K and SYMM cases shared by the oracle tests, the golden-vector generator and the GPU parity
tests; same conventions as tests/cases.py.  Whatever a routine must not read or write holds NaN: the
unreferenced triangle of C (SYR2K) and of the symmetric matrix A (SYMM)."""
from __future__ import annotations

import itertools

import numpy as np

import oracle
from oracle import ConjTrans, Left, Lower, NoTrans, Right, Trans, Upper
from tests.cases import DT, ORDERS, _min_ld


def _draw(g, mode, shape, dt):
    if mode == "int":
        return g.integers(-8, 9, size=shape).astype(dt)
    return g.uniform(-1, 1, size=shape).astype(dt)


def other_triangle(n, uplo):
    """Boolean mask of the strict triangle that `uplo` does not reference."""
    return np.triu(np.ones((n, n), dtype=bool), 1) if uplo == Lower else np.tril(np.ones((n, n), dtype=bool), -1)


# ------------------------------------------------------------------------------------------- SYR2K
def syr2k_case(prec, order, uplo, trans, N, K, alpha=1.0, beta=1.0, pad=(0, 0, 0), off=(0, 0, 0), mode="int", seed=12345):
    ld = _min_ld(order, trans, N, K)
    return dict(kind="syr2k", prec=prec, order=order, uplo=uplo, trans=trans, N=N, K=K, alpha=alpha, beta=beta,
                lda=ld + pad[0], ldb=ld + pad[1], ldc=N + pad[2], offA=off[0], offB=off[1], offC=off[2], mode=mode, seed=seed)


def syr2k_logical(c):
    dt = DT[c["prec"]]
    g = oracle.rng(c["seed"], 29)
    N, K = c["N"], c["K"]
    opA, opB, C = _draw(g, c["mode"], (N, K), dt), _draw(g, c["mode"], (N, K), dt), _draw(g, c["mode"], (N, N), dt)
    C[other_triangle(N, c["uplo"])] = np.nan
    return opA, opB, C


def syr2k_buffers(c, logical=None, tail=3):
    opA, opB, C = logical if logical is not None else syr2k_logical(c)
    return (oracle.pack(opA, c["order"], c["trans"], c["lda"], c["offA"], tail=tail),
            oracle.pack(opB, c["order"], c["trans"], c["ldb"], c["offB"], tail=tail),
            oracle.pack(C, c["order"], NoTrans, c["ldc"], c["offC"], tail=tail))


def golden_syr2k_cases():
    out = {}
    k = 0
    for prec in "sd":
        for order, uplo, tr in itertools.product(ORDERS, (Upper, Lower), (NoTrans, Trans)):
            N, K = [(9, 5), (16, 17), (33, 12)][k % 3]
            out[f"syr2k_{prec}_{order}{uplo}{tr}"] = syr2k_case(prec, order, uplo, tr, N, K, alpha=[1.0, -2.0, 0.5][k % 3],
                                                              beta=[0.5, 0.0, 3.0][k % 3], pad=(2, 1, 3), off=(1, 2, 4),
                                                              mode=["int", "uniform"][k % 2], seed=700 + k)
            k += 1
    return out


def sweep_syr2k_cases(prec, mode):
    cases = []
    seed = 9000
    for order, uplo, tr in itertools.product(ORDERS, (Upper, Lower), (NoTrans, Trans, ConjTrans)):
        for (N, K) in ((8, 8), (17, 33), (128, 64), (257, 130), (300, 129), (700, 96)):
            seed += 1
            cases.append(syr2k_case(prec, order, uplo, tr, N, K, alpha=[1.0, 2.0, -3.0][seed % 3], beta=[1.0, 0.0, 2.0][seed % 3],
                                    pad=(seed % 5, seed % 3, seed % 7), off=(seed % 3, seed % 5, seed % 11), mode=mode, seed=seed))
    return cases


# -------------------------------------------------------------------------------------------- SYMM
def symm_case(prec, order, side, uplo, M, N, alpha=1.0, beta=1.0, pad=(0, 0, 0), off=(0, 0, 0), mode="int", seed=12345):
    n = M if side == Left else N
    ldbc = _min_ld(order, NoTrans, M, N)
    return dict(kind="symm", prec=prec, order=order, side=side, uplo=uplo, M=M, N=N, alpha=alpha, beta=beta,
                lda=n + pad[0], ldb=ldbc + pad[1], ldc=ldbc + pad[2], offA=off[0], offB=off[1], offC=off[2], mode=mode, seed=seed)


def symm_logical(c):
    """(A with NaN in the triangle that is not stored, the dense symmetric matrix it stands for, B, C)."""
    dt = DT[c["prec"]]
    g = oracle.rng(c["seed"], 31)
    M, N = c["M"], c["N"]
    n = M if c["side"] == Left else N
    R = _draw(g, c["mode"], (n, n), dt)
    full = np.tril(R) + np.tril(R, -1).T
    A = full.copy()
    A[other_triangle(n, c["uplo"])] = np.nan
    return A, full, _draw(g, c["mode"], (M, N), dt), _draw(g, c["mode"], (M, N), dt)


def symm_buffers(c, logical=None, tail=3):
    A, _, B, C = logical if logical is not None else symm_logical(c)
    return (oracle.pack(A, c["order"], NoTrans, c["lda"], c["offA"], tail=tail),
            oracle.pack(B, c["order"], NoTrans, c["ldb"], c["offB"], tail=tail),
            oracle.pack(C, c["order"], NoTrans, c["ldc"], c["offC"], tail=tail))


def symm_exact(c, logical):
    """float64 value of alpha*A*B + beta*C (or B*A) and the magnitude sum that scales the error bound."""
    _, full, B, C = (x.astype(np.float64) for x in logical)
    if c["side"] == Left:
        return c["alpha"] * (full @ B) + c["beta"] * C, abs(c["alpha"]) * (np.abs(full) @ np.abs(B)) + abs(c["beta"]) * np.abs(C)
    return c["alpha"] * (B @ full) + c["beta"] * C, abs(c["alpha"]) * (np.abs(B) @ np.abs(full)) + abs(c["beta"]) * np.abs(C)


def golden_symm_cases():
    out = {}
    k = 0
    for prec in "sd":
        for order, side, uplo in itertools.product(ORDERS, (Left, Right), (Upper, Lower)):
            M, N = [(9, 5), (16, 17), (12, 33)][k % 3]
            out[f"symm_{prec}_{order}{side}{uplo}"] = symm_case(prec, order, side, uplo, M, N, alpha=[1.0, -2.0, 0.5][k % 3],
                                                              beta=[0.5, 0.0, 3.0][k % 3], pad=(2, 1, 3), off=(1, 2, 4),
                                                              mode=["int", "uniform"][k % 2], seed=800 + k)
            k += 1
    return out


def sweep_symm_cases(prec, mode):
    cases = []
    seed = 9500
    for order, side, uplo in itertools.product(ORDERS, (Left, Right), (Upper, Lower)):
        for (M, N) in ((8, 8), (17, 33), (128, 64), (257, 130), (130, 300), (700, 96), (96, 515)):
            seed += 1
            cases.append(symm_case(prec, order, side, uplo, M, N, alpha=[1.0, 2.0, -3.0][seed % 3], beta=[1.0, 0.0, 2.0][seed % 3],
                                   pad=(seed % 5, seed % 3, seed % 7), off=(seed % 3, seed % 5, seed % 11), mode=mode, seed=seed))
    return cases
