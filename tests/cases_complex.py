"""Seeded complex GEMM cases (clblasCgemm / clblasZgemm) shared by the oracle tests, the golden-vector
generator and the GPU parity tests; same conventions as tests/cases.py.  A logical op(X) that was
produced by ConjTrans is stored conjugated, so that reading it back through ConjTrans gives op(X)."""
from __future__ import annotations

import itertools

import numpy as np

import oracle
from oracle import ConjTrans, NoTrans, Trans
from tests.cases import ORDERS, _min_ld

CDT = {"c": np.complex64, "z": np.complex128}
RDT = {"c": np.float32, "z": np.float64}
CNAN = complex(np.nan, np.nan)
ALL_TRANS = (NoTrans, Trans, ConjTrans)


def cgemm_case(prec, order, transA, transB, M, N, K, alpha=1.5 - 0.5j, beta=0.5 + 0.25j, pad=(0, 0, 0), off=(0, 0, 0),
               mode="uniform", seed=12345):
    return dict(kind="cgemm", prec=prec, order=order, transA=transA, transB=transB, M=M, N=N, K=K, alpha=alpha, beta=beta,
                lda=_min_ld(order, transA, M, K) + pad[0], ldb=_min_ld(order, transB, K, N) + pad[1],
                ldc=_min_ld(order, NoTrans, M, N) + pad[2], offA=off[0], offB=off[1], offC=off[2], mode=mode, seed=seed)


def _draw(g, mode, shape, prec):
    if mode == "int":
        re, im = g.integers(-6, 7, size=shape), g.integers(-6, 7, size=shape)
    else:
        re, im = g.uniform(-1, 1, size=shape), g.uniform(-1, 1, size=shape)
    return (re + 1j * im).astype(CDT[prec])


def cgemm_logical(c):
    """Logical op(A) (M x K), op(B) (K x N) and C (M x N)."""
    g = oracle.rng(c["seed"], 37)
    return (_draw(g, c["mode"], (c["M"], c["K"]), c["prec"]), _draw(g, c["mode"], (c["K"], c["N"]), c["prec"]),
            _draw(g, c["mode"], (c["M"], c["N"]), c["prec"]))


def cgemm_buffers(c, logical=None, tail=3):
    opA, opB, C = logical if logical is not None else cgemm_logical(c)
    sA = np.conj(opA) if c["transA"] == ConjTrans else opA
    sB = np.conj(opB) if c["transB"] == ConjTrans else opB
    return (oracle.pack(sA, c["order"], c["transA"], c["lda"], c["offA"], pad_value=CNAN, tail=tail),
            oracle.pack(sB, c["order"], c["transB"], c["ldb"], c["offB"], pad_value=CNAN, tail=tail),
            oracle.pack(C, c["order"], NoTrans, c["ldc"], c["offC"], pad_value=CNAN, tail=tail))


def cgemm_exact(c, logical):
    """complex128 value of alpha*op(A)*op(B) + beta*C and the magnitude sum that scales the error bound."""
    opA, opB, C = (x.astype(np.complex128) for x in logical)
    want = c["alpha"] * (opA @ opB) + c["beta"] * C
    mag = abs(c["alpha"]) * (np.abs(opA) @ np.abs(opB)) + abs(c["beta"]) * np.abs(C)
    return want, mag


def golden_cgemm_cases():
    out = {}
    k = 0
    for prec in "cz":
        for order, ta, tb in itertools.product(ORDERS, ALL_TRANS, ALL_TRANS):
            M, N, K = [(17, 13, 9), (32, 8, 33), (5, 62, 16), (64, 17, 8)][k % 4]
            out[f"cgemm_{prec}_{order}{ta}{tb}"] = cgemm_case(prec, order, ta, tb, M, N, K, alpha=[2 - 1j, 1.5 + 0.5j][k % 2],
                                                             beta=[3 + 0j, 0.5 - 2j, 0j][k % 3], pad=(3, 1, 2), off=(5, 2, 7),
                                                             mode=["int", "uniform"][k % 2], seed=1100 + k)
            k += 1
    return out


def sweep_cgemm_cases(prec, mode):
    cases = []
    seed = 12000
    for order in ORDERS:
        for ta, tb in itertools.product(ALL_TRANS, ALL_TRANS):
            for (M, N, K) in ((8, 8, 8), (17, 17, 17), (64, 62, 144), (128, 144, 17), (129, 257, 65), (300, 200, 130)):
                seed += 1
                cases.append(cgemm_case(prec, order, ta, tb, M, N, K, alpha=[1 + 0j, 2 - 1j, -1 + 3j][seed % 3],
                                        beta=[1 + 0j, 0j, 2 + 1j, -1 + 0j][seed % 4], pad=(seed % 4, seed % 3, seed % 5),
                                        off=(seed % 3, seed % 4, seed % 6), mode=mode, seed=seed))
    return cases


# ------------------------------------------------------------------------------------- complex TRSM
from oracle import Left, Lower, NonUnit, Right, Unit, Upper  # noqa: E402


def ctrsm_case(prec, order, side, uplo, transA, diag, M, N, alpha=1 + 0j, pad=(0, 0), off=(0, 0), seed=12345):
    n = M if side == Left else N
    return dict(kind="ctrsm", prec=prec, order=order, side=side, uplo=uplo, transA=transA, diag=diag, M=M, N=N, alpha=alpha,
                lda=n + pad[0], ldb=_min_ld(order, NoTrans, M, N) + pad[1], offA=off[0], offB=off[1], seed=seed)


def ctrsm_logical(c):
    """Stored triangular A (n x n complex; NaN outside the referenced triangle and on a unit diagonal) and B.
    Real and imaginary parts each follow the reference-style generator of the real TRSM cases, so rows
    stay diagonally dominant."""
    n = c["M"] if c["side"] == Left else c["N"]
    rd = RDT[c["prec"]]
    Ar, Br = oracle.trsm_inputs(n, (c["M"], c["N"]), c["uplo"], c["diag"], rd, c["seed"])
    Ai, Bi = oracle.trsm_inputs(n, (c["M"], c["N"]), c["uplo"], c["diag"], rd, c["seed"] + 7919)
    return (Ar + 1j * (Ai / 2)).astype(CDT[c["prec"]]), (Br + 1j * Bi).astype(CDT[c["prec"]])


def ctrsm_buffers(c, logical=None, tail=3):
    A, B = logical if logical is not None else ctrsm_logical(c)
    return (oracle.pack(A, c["order"], NoTrans, c["lda"], c["offA"], pad_value=CNAN, tail=tail),
            oracle.pack(B, c["order"], NoTrans, c["ldb"], c["offB"], pad_value=CNAN, tail=tail))


def ctrsm_op_triangle(c, A):
    """Dense op(A): zeros outside the triangle, ones on a unit diagonal, transposed / conjugated as asked."""
    T = np.tril(np.nan_to_num(A, nan=0.0)) if c["uplo"] == Lower else np.triu(np.nan_to_num(A, nan=0.0))
    if c["diag"] == Unit:
        T = T.copy()
        T[np.arange(T.shape[0]), np.arange(T.shape[0])] = 1.0
    return T if c["transA"] == NoTrans else (T.T if c["transA"] == Trans else np.conj(T.T))


def ctrsm_backward_ratio(c, X, T, B):
    """max |alpha B - op(A) X| / (|op(A)||X| + |alpha||B|) (X op(A) for Right), divided by 4*(2n)*u."""
    T, X, B = (x.astype(np.complex128) for x in (T, X, B))
    if c["side"] == Left:
        res, den = c["alpha"] * B - T @ X, np.abs(T) @ np.abs(X) + abs(c["alpha"]) * np.abs(B)
    else:
        res, den = c["alpha"] * B - X @ T, np.abs(X) @ np.abs(T) + abs(c["alpha"]) * np.abs(B)
    den = np.where(den == 0, np.finfo(np.float64).tiny, den)
    return float(np.max(np.abs(res) / den) / (4.0 * 2 * T.shape[0] * oracle.unit_roundoff(RDT[c["prec"]])))


def golden_ctrsm_cases():
    out = {}
    k = 0
    for prec in "cz":
        for order, side, uplo, ta, diag in itertools.product(ORDERS, (Left, Right), (Upper, Lower), ALL_TRANS, (Unit, NonUnit)):
            M, N = [(9, 5), (16, 17), (7, 12)][k % 3]
            out[f"ctrsm_{prec}_{order}{side}{uplo}{ta}{diag}"] = ctrsm_case(prec, order, side, uplo, ta, diag, M, N,
                                                                           alpha=[1 + 0j, -2 + 1j, 0.5j][k % 3], pad=(2, 3),
                                                                           off=(1, 4), seed=1300 + k)
            k += 1
    return out


def sweep_ctrsm_cases(prec):
    cases = []
    seed = 14000
    for order, side, uplo, ta, diag in itertools.product(ORDERS, (Left, Right), (Upper, Lower), ALL_TRANS, (Unit, NonUnit)):
        for (M, N) in ((8, 8), (17, 33), (64, 64), (130, 257), (300, 129)):
            seed += 1
            cases.append(ctrsm_case(prec, order, side, uplo, ta, diag, M, N, alpha=[1 + 0j, 2.5 - 1j, -0.5j][seed % 3],
                                    pad=(seed % 5, seed % 7), off=(seed % 3, seed % 11), seed=seed))
    return cases


# ------------------------------------------------- complex SYRK / HERK / SYR2K / HER2K / SYMM / HEMM
def _other_triangle(n, uplo):
    return np.triu(np.ones((n, n), dtype=bool), 1) if uplo == Lower else np.tril(np.ones((n, n), dtype=bool), -1)


def crank_case(kind, prec, order, uplo, trans, N, K, alpha, beta, pad=(0, 0, 0), off=(0, 0, 0), mode="int", seed=12345):
    """kind: syrk | herk | syr2k | her2k.  trans: NoTrans, or Trans (symmetric kinds) / ConjTrans (Hermitian kinds)."""
    ld = _min_ld(order, trans, N, K)
    return dict(kind=kind, prec=prec, order=order, uplo=uplo, trans=trans, N=N, K=K, alpha=alpha, beta=beta,
                lda=ld + pad[0], ldb=ld + pad[1], ldc=N + pad[2], offA=off[0], offB=off[1], offC=off[2], mode=mode, seed=seed)


def crank_logical(c):
    """op(A), op(B) (N x K) and C (N x N: NaN in the triangle that is not referenced; real diagonal for Hermitian kinds)."""
    g = oracle.rng(c["seed"], 41)
    opA = _draw(g, c["mode"], (c["N"], c["K"]), c["prec"])
    opB = _draw(g, c["mode"], (c["N"], c["K"]), c["prec"])
    C = _draw(g, c["mode"], (c["N"], c["N"]), c["prec"])
    if c["kind"] in ("herk", "her2k"):
        C[np.arange(c["N"]), np.arange(c["N"])] = C.diagonal().real
    C[_other_triangle(c["N"], c["uplo"])] = CNAN
    return opA, opB, C


def crank_buffers(c, logical=None, tail=3):
    opA, opB, C = logical if logical is not None else crank_logical(c)
    herm = c["kind"] in ("herk", "her2k")
    # the stored matrix X satisfies op(X) = opX: X = opX, opX^T, or conj(opX)^T when op is the conjugate transposition
    sA = np.conj(opA) if (herm and c["trans"] != NoTrans) else opA
    sB = np.conj(opB) if (herm and c["trans"] != NoTrans) else opB
    return (oracle.pack(sA, c["order"], c["trans"], c["lda"], c["offA"], pad_value=CNAN, tail=tail),
            oracle.pack(sB, c["order"], c["trans"], c["ldb"], c["offB"], pad_value=CNAN, tail=tail),
            oracle.pack(C, c["order"], NoTrans, c["ldc"], c["offC"], pad_value=CNAN, tail=tail))


def crank_exact(c, logical):
    """complex128 value of the update on the whole matrix and the magnitude sum that scales the error bound."""
    opA, opB, C = (x.astype(np.complex128) for x in logical)
    C = np.nan_to_num(C)
    a, b = c["alpha"], c["beta"]
    k = c["kind"]
    if k == "syrk":
        want, mag = a * (opA @ opA.T) + b * C, abs(a) * (np.abs(opA) @ np.abs(opA).T) + abs(b) * np.abs(C)
    elif k == "herk":
        want, mag = a * (opA @ opA.conj().T) + b * C, abs(a) * (np.abs(opA) @ np.abs(opA).T) + abs(b) * np.abs(C)
    elif k == "syr2k":
        want = a * (opA @ opB.T + opB @ opA.T) + b * C
        mag = abs(a) * (np.abs(opA) @ np.abs(opB).T + np.abs(opB) @ np.abs(opA).T) + abs(b) * np.abs(C)
    else:
        want = a * (opA @ opB.conj().T) + np.conj(a) * (opB @ opA.conj().T) + b * C
        mag = abs(a) * (np.abs(opA) @ np.abs(opB).T + np.abs(opB) @ np.abs(opA).T) + abs(b) * np.abs(C)
    if k in ("herk", "her2k"):
        want = want.copy()
        want[np.arange(c["N"]), np.arange(c["N"])] = want.diagonal().real
    return want, mag


def crank_scalars(kind, k):
    if kind == "syrk":
        return [1 + 0j, 2 - 1j, -1 + 3j][k % 3], [1 + 0j, 0j, 2 + 1j][k % 3]
    if kind == "herk":
        return [1.0, 2.0, -3.0][k % 3], [1.0, 0.0, 2.0][k % 3]
    if kind == "syr2k":
        return [1 + 0j, 2 - 1j, -1 + 3j][k % 3], [1 + 0j, 0j, 2 + 1j][k % 3]
    return [1 + 0j, 2 - 1j, -1 + 3j][k % 3], [1.0, 0.0, 2.0][k % 3]


def golden_crank_cases():
    out = {}
    k = 0
    for kind in ("syrk", "herk", "syr2k", "her2k"):
        t2 = Trans if kind in ("syrk", "syr2k") else ConjTrans
        for prec in "cz":
            for order, uplo, tr in itertools.product(ORDERS, (Upper, Lower), (NoTrans, t2)):
                N, K = [(9, 5), (16, 17), (33, 12)][k % 3]
                al, be = crank_scalars(kind, k)
                out[f"c{kind}_{prec}_{order}{uplo}{tr}"] = crank_case(kind, prec, order, uplo, tr, N, K, al, be, pad=(2, 1, 3),
                                                                    off=(1, 2, 4), mode=["int", "uniform"][k % 2], seed=1500 + k)
                k += 1
    return out


def sweep_crank_cases(kind, prec, mode):
    cases = []
    seed = 16000
    t2 = Trans if kind in ("syrk", "syr2k") else ConjTrans
    for order, uplo, tr in itertools.product(ORDERS, (Upper, Lower), (NoTrans, t2)):
        for (N, K) in ((8, 8), (17, 33), (128, 64), (257, 130), (300, 129)):
            seed += 1
            al, be = crank_scalars(kind, seed)
            cases.append(crank_case(kind, prec, order, uplo, tr, N, K, al, be, pad=(seed % 5, seed % 3, seed % 7),
                                    off=(seed % 3, seed % 5, seed % 11), mode=mode, seed=seed))
    return cases


def csymm_case(kind, prec, order, side, uplo, M, N, alpha, beta, pad=(0, 0, 0), off=(0, 0, 0), mode="int", seed=12345):
    """kind: symm | hemm."""
    n = M if side == Left else N
    ldbc = _min_ld(order, NoTrans, M, N)
    return dict(kind=kind, prec=prec, order=order, side=side, uplo=uplo, M=M, N=N, alpha=alpha, beta=beta,
                lda=n + pad[0], ldb=ldbc + pad[1], ldc=ldbc + pad[2], offA=off[0], offB=off[1], offC=off[2], mode=mode, seed=seed)


def csymm_logical(c):
    """(stored A with NaN in the other triangle -- and, for HEMM, garbage imaginary parts on the diagonal, which must be
    ignored -- the dense matrix it stands for, B, C)."""
    g = oracle.rng(c["seed"], 43)
    n = c["M"] if c["side"] == Left else c["N"]
    R = _draw(g, c["mode"], (n, n), c["prec"])
    if c["kind"] == "hemm":
        full = np.tril(R, -1) + np.tril(R, -1).conj().T + np.diag(R.diagonal().real)
    else:
        full = np.tril(R) + np.tril(R, -1).T
    full = full.astype(CDT[c["prec"]])
    A = full.copy()
    if c["kind"] == "hemm":
        A[np.arange(n), np.arange(n)] = full.diagonal().real + 1j * 7.0
    A[_other_triangle(n, c["uplo"])] = CNAN
    return A, full, _draw(g, c["mode"], (c["M"], c["N"]), c["prec"]), _draw(g, c["mode"], (c["M"], c["N"]), c["prec"])


def csymm_buffers(c, logical=None, tail=3):
    A, _, B, C = logical if logical is not None else csymm_logical(c)
    return (oracle.pack(A, c["order"], NoTrans, c["lda"], c["offA"], pad_value=CNAN, tail=tail),
            oracle.pack(B, c["order"], NoTrans, c["ldb"], c["offB"], pad_value=CNAN, tail=tail),
            oracle.pack(C, c["order"], NoTrans, c["ldc"], c["offC"], pad_value=CNAN, tail=tail))


def csymm_exact(c, logical):
    _, full, B, C = (x.astype(np.complex128) for x in logical)
    a, b = c["alpha"], c["beta"]
    if c["side"] == Left:
        return a * (full @ B) + b * C, abs(a) * (np.abs(full) @ np.abs(B)) + abs(b) * np.abs(C)
    return a * (B @ full) + b * C, abs(a) * (np.abs(B) @ np.abs(full)) + abs(b) * np.abs(C)


def golden_csymm_cases():
    out = {}
    k = 0
    for kind in ("symm", "hemm"):
        for prec in "cz":
            for order, side, uplo in itertools.product(ORDERS, (Left, Right), (Upper, Lower)):
                M, N = [(9, 5), (16, 17), (12, 33)][k % 3]
                out[f"c{kind}_{prec}_{order}{side}{uplo}"] = csymm_case(kind, prec, order, side, uplo, M, N, [1 + 0j, -2 + 1j, 0.5j][k % 3],
                                                                      [0.5 + 0j, 0j, 3 - 1j][k % 3], pad=(2, 1, 3), off=(1, 2, 4),
                                                                      mode=["int", "uniform"][k % 2], seed=1700 + k)
                k += 1
    return out


def sweep_csymm_cases(kind, prec, mode):
    cases = []
    seed = 17000
    for order, side, uplo in itertools.product(ORDERS, (Left, Right), (Upper, Lower)):
        for (M, N) in ((8, 8), (17, 33), (128, 64), (257, 130), (130, 300)):
            seed += 1
            cases.append(csymm_case(kind, prec, order, side, uplo, M, N, [1 + 0j, 2 - 1j, -3j][seed % 3], [1 + 0j, 0j, 2 + 1j][seed % 3],
                                    pad=(seed % 5, seed % 3, seed % 7), off=(seed % 3, seed % 5, seed % 11), mode=mode, seed=seed))
    return cases


# ------------------------------------------------------------------------------------- complex TRMM
def ctrmm_case(prec, order, side, uplo, transA, diag, M, N, alpha=1 + 0j, pad=(0, 0), off=(0, 0), mode="int", seed=12345):
    n = M if side == Left else N
    return dict(kind="ctrmm", prec=prec, order=order, side=side, uplo=uplo, transA=transA, diag=diag, M=M, N=N, alpha=alpha,
                lda=n + pad[0], ldb=_min_ld(order, NoTrans, M, N) + pad[1], offA=off[0], offB=off[1], mode=mode, seed=seed)


def ctrmm_logical(c):
    """Stored triangular A (NaN outside the referenced triangle and on a unit diagonal) and B."""
    g = oracle.rng(c["seed"], 47)
    n = c["M"] if c["side"] == Left else c["N"]
    A = _draw(g, c["mode"], (n, n), c["prec"])
    A[_other_triangle(n, c["uplo"])] = CNAN
    if c["diag"] == Unit:
        A[np.arange(n), np.arange(n)] = CNAN
    return A, _draw(g, c["mode"], (c["M"], c["N"]), c["prec"])


def ctrmm_buffers(c, logical=None, tail=3):
    A, B = logical if logical is not None else ctrmm_logical(c)
    return (oracle.pack(A, c["order"], NoTrans, c["lda"], c["offA"], pad_value=CNAN, tail=tail),
            oracle.pack(B, c["order"], NoTrans, c["ldb"], c["offB"], pad_value=CNAN, tail=tail))


def ctrmm_exact(c, logical):
    A, B = logical
    T = ctrsm_op_triangle(c, A).astype(np.complex128)
    B = B.astype(np.complex128)
    if c["side"] == Left:
        return c["alpha"] * (T @ B), abs(c["alpha"]) * (np.abs(T) @ np.abs(B)), T
    return c["alpha"] * (B @ T), abs(c["alpha"]) * (np.abs(B) @ np.abs(T)), T


def golden_ctrmm_cases():
    out = {}
    k = 0
    for prec in "cz":
        for order, side, uplo, ta, diag in itertools.product(ORDERS, (Left, Right), (Upper, Lower), ALL_TRANS, (Unit, NonUnit)):
            M, N = [(9, 5), (16, 17), (7, 12)][k % 3]
            out[f"ctrmm_{prec}_{order}{side}{uplo}{ta}{diag}"] = ctrmm_case(prec, order, side, uplo, ta, diag, M, N,
                                                                           alpha=[1 + 0j, -2 + 1j, 0.5j][k % 3], pad=(2, 3), off=(1, 4),
                                                                           mode=["int", "uniform"][k % 2], seed=1900 + k)
            k += 1
    return out


def sweep_ctrmm_cases(prec, mode):
    cases = []
    seed = 19000
    for order, side, uplo, ta, diag in itertools.product(ORDERS, (Left, Right), (Upper, Lower), ALL_TRANS, (Unit, NonUnit)):
        for (M, N) in ((8, 8), (17, 33), (64, 64), (130, 257), (300, 129)):
            seed += 1
            cases.append(ctrmm_case(prec, order, side, uplo, ta, diag, M, N, alpha=[1 + 0j, 2 - 1j, -3j][seed % 3],
                                    pad=(seed % 5, seed % 7), off=(seed % 3, seed % 11), mode=mode, seed=seed))
    return cases
