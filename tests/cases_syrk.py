"""Seeded SYRK cases (C <- alpha*op(A)*op(A)^T + beta*C on one triangle) shared by the oracle tests, the
golden-vector generator and the GPU parity tests; same conventions as tests/cases.py.  The triangle
of C that must not be touched holds NaN."""
from __future__ import annotations

import itertools

import numpy as np

import oracle
from oracle import ColumnMajor, Lower, NoTrans, RowMajor, Trans, ConjTrans, Upper
from tests.cases import DT, ORDERS, _min_ld


def syrk_case(prec, order, uplo, trans, N, K, alpha=1.0, beta=1.0, pad=(0, 0), off=(0, 0), mode="int", seed=12345):
    return dict(kind="syrk", prec=prec, order=order, uplo=uplo, trans=trans, N=N, K=K, alpha=alpha, beta=beta,
                lda=_min_ld(order, trans, N, K) + pad[0], ldc=N + pad[1], offA=off[0], offC=off[1], mode=mode, seed=seed)


def syrk_logical(c):
    """op(A) (N x K) and C (N x N, NaN in the triangle that is not referenced)."""
    dt = DT[c["prec"]]
    g = oracle.rng(c["seed"], 23)
    N, K = c["N"], c["K"]
    if c["mode"] == "int":
        opA = g.integers(-8, 9, size=(N, K)).astype(dt)
        C = g.integers(-8, 9, size=(N, N)).astype(dt)
    else:
        opA = g.uniform(-1, 1, size=(N, K)).astype(dt)
        C = g.uniform(-1, 1, size=(N, N)).astype(dt)
    mask = np.triu(np.ones((N, N), dtype=bool), 1) if c["uplo"] == Lower else np.tril(np.ones((N, N), dtype=bool), -1)
    C[mask] = np.nan
    return opA, C


def syrk_buffers(c, logical=None, tail=3):
    opA, C = logical if logical is not None else syrk_logical(c)
    return (oracle.pack(opA, c["order"], c["trans"], c["lda"], c["offA"], tail=tail),
            oracle.pack(C, c["order"], NoTrans, c["ldc"], c["offC"], tail=tail))


def golden_syrk_cases():
    out = {}
    k = 0
    for prec in "sd":
        for order, uplo, tr in itertools.product(ORDERS, (Upper, Lower), (NoTrans, Trans)):
            N, K = [(9, 5), (16, 17), (33, 12)][k % 3]
            out[f"syrk_{prec}_{order}{uplo}{tr}"] = syrk_case(prec, order, uplo, tr, N, K, alpha=[1.0, -2.0, 0.5][k % 3],
                                                            beta=[0.5, 0.0, 3.0][k % 3], pad=(2, 3), off=(1, 4),
                                                            mode=["int", "uniform"][k % 2], seed=600 + k)
            k += 1
    return out


def sweep_syrk_cases(prec, mode):
    cases = []
    seed = 8000
    for order, uplo, tr in itertools.product(ORDERS, (Upper, Lower), (NoTrans, Trans, ConjTrans)):
        for (N, K) in ((8, 8), (17, 33), (128, 64), (257, 130), (300, 129), (700, 96)):
            seed += 1
            cases.append(syrk_case(prec, order, uplo, tr, N, K, alpha=[1.0, 2.0, -3.0][seed % 3], beta=[1.0, 0.0, 2.0][seed % 3],
                                   pad=(seed % 5, seed % 7), off=(seed % 3, seed % 11), mode=mode, seed=seed))
    return cases
