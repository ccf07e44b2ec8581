"""Generates tests/golden/level3_golden.npz from the reference's own CPU BLAS.

Run in a container that holds the reference tree (it needs oracle/_ref/libnaive_ref.so, which
oracle/Makefile builds from the reference's src/library/tools/ktest/naive/naive_blas.cpp):

    python tests/golden/make_golden.py

Each case stores the seeded inputs' parameters and the output buffer NaiveBlas produced, so
that on a machine without the reference tree the C restatement (and the CUDA path) can still
be checked against the reference's results.  Inputs are regenerated from the seed by
tests/cases.py; only outputs are stored.
"""
import os
import sys

import numpy as np

sys.path.insert(0, os.path.join(os.path.dirname(__file__), "..", ".."))
import oracle  # noqa: E402
from tests import cases, cases_complex, cases_sym, cases_syrk, cases_trmm  # noqa: E402


def symm_by_external_blas(c):
    """C buffer after ?symm of the Netlib interface (scipy.linalg.blas); B and C go in as column-major views."""
    from scipy.linalg import blas
    from oracle import Left, Lower, NoTrans
    logical = cases_sym.symm_logical(c)
    A, full, B, C = logical
    fn = blas.ssymm if c["prec"] == "s" else blas.dsymm
    stored = np.where(np.isnan(A), 0, A)      # Fortran symm reads only the uplo triangle
    R = fn(c["alpha"], np.asfortranarray(stored), np.asfortranarray(B), beta=c["beta"], c=np.asfortranarray(C),
           side=0 if c["side"] == Left else 1, lower=1 if c["uplo"] == Lower else 0)
    return oracle.pack(np.ascontiguousarray(R), c["order"], NoTrans, c["ldc"], c["offC"], tail=3)


def hermitian_update_by_external_blas(c):
    """Logical N x N result of ?herk / ?her2k of the Netlib interface (scipy.linalg.blas) on the logical operands; the
    triangle that is not referenced keeps the input's NaN."""
    from scipy.linalg import blas
    from oracle import Lower, NoTrans
    opA, opB, C = cases_complex.crank_logical(c)
    z = c["prec"] == "z"
    C0 = np.nan_to_num(C)
    lower = 1 if c["uplo"] == Lower else 0
    # the operands are handed over as op(X) itself (trans = 0): what is tested downstream is the definition
    if c["kind"] == "herk":
        fn = blas.zherk if z else blas.cherk
        R = fn(c["alpha"], np.asfortranarray(opA), beta=c["beta"], c=np.asfortranarray(C0), trans=0, lower=lower)
    else:
        fn = blas.zher2k if z else blas.cher2k
        R = fn(c["alpha"], np.asfortranarray(opA), np.asfortranarray(opB), beta=c["beta"], c=np.asfortranarray(C0), trans=0,
               lower=lower)
    R = np.array(R)
    R[cases_complex._other_triangle(c["N"], c["uplo"])] = cases_complex.CNAN
    return R


def complex_symm_by_external_blas(c):
    from scipy.linalg import blas
    from oracle import Left, Lower
    A, full, B, C = cases_complex.csymm_logical(c)
    z = c["prec"] == "z"
    fn = {("symm", True): blas.zsymm, ("symm", False): blas.csymm, ("hemm", True): blas.zhemm, ("hemm", False): blas.chemm}[(c["kind"], z)]
    stored = np.where(np.isnan(A), 0, A)
    return np.array(fn(c["alpha"], np.asfortranarray(stored), np.asfortranarray(B), beta=c["beta"], c=np.asfortranarray(C),
                       side=0 if c["side"] == Left else 1, lower=1 if c["uplo"] == Lower else 0))


def main():
    oracle.build()
    assert oracle.have_ref(), "oracle/_ref/libnaive_ref.so missing: reference tree not present"
    out = {}
    for name, c in cases.golden_gemm_cases().items():
        A, B, C = cases.gemm_buffers(c)
        oracle.gemm(c["order"], c["transA"], c["transB"], c["M"], c["N"], c["K"], c["alpha"], A, c["offA"],
                    c["lda"], B, c["offB"], c["ldb"], c["beta"], C, c["offC"], c["ldc"], impl="ref")
        out[name] = C
    for name, c in cases.golden_trsm_cases().items():
        A, B = cases.trsm_buffers(c)
        oracle.trsm(c["order"], c["side"], c["uplo"], c["transA"], c["diag"], c["M"], c["N"], c["alpha"], A,
                    c["offA"], c["lda"], B, c["offB"], c["ldb"], impl="ref")
        out[name] = B
    for name, c in cases_trmm.golden_trmm_cases().items():
        A, B = cases_trmm.trmm_buffers(c)
        oracle.trmm(c["order"], c["side"], c["uplo"], c["transA"], c["diag"], c["M"], c["N"], c["alpha"], A,
                    c["offA"], c["lda"], B, c["offB"], c["ldb"], impl="ref")
        out[name] = B
    for name, c in cases_syrk.golden_syrk_cases().items():
        A, C = cases_syrk.syrk_buffers(c)
        oracle.syrk(c["order"], c["uplo"], c["trans"], c["N"], c["K"], c["alpha"], A, c["offA"], c["lda"], c["beta"], C,
                    c["offC"], c["ldc"], impl="ref")
        out[name] = C
    for name, c in cases_sym.golden_syr2k_cases().items():
        A, B, C = cases_sym.syr2k_buffers(c)
        oracle.syr2k(c["order"], c["uplo"], c["trans"], c["N"], c["K"], c["alpha"], A, c["offA"], c["lda"], B, c["offB"],
                     c["ldb"], c["beta"], C, c["offC"], c["ldc"], impl="ref")
        out[name] = C
    # SYMM: the reference's naive BLAS has none and its tests call an external Fortran BLAS, so these
    # vectors come from that interface here (OpenBLAS through scipy), on the dense symmetric matrix
    for name, c in cases_sym.golden_symm_cases().items():
        out[name] = symm_by_external_blas(c)
    for name, c in cases_complex.golden_cgemm_cases().items():
        A, B, C = cases_complex.cgemm_buffers(c)
        oracle.cgemm(c["order"], c["transA"], c["transB"], c["M"], c["N"], c["K"], c["alpha"], A, c["offA"], c["lda"],
                     B, c["offB"], c["ldb"], c["beta"], C, c["offC"], c["ldc"], impl="ref")
        out[name] = C
    for name, c in cases_complex.golden_ctrsm_cases().items():
        A, B = cases_complex.ctrsm_buffers(c)
        oracle.ctrsm(c["order"], c["side"], c["uplo"], c["transA"], c["diag"], c["M"], c["N"], c["alpha"], A, c["offA"],
                     c["lda"], B, c["offB"], c["ldb"], impl="ref")
        out[name] = B
    cc = cases_complex
    for name, c in cc.golden_crank_cases().items():
        if c["kind"] in ("syrk", "syr2k"):
            A, B, C = cc.crank_buffers(c)
            if c["kind"] == "syrk":
                oracle.csyrk(c["order"], c["uplo"], c["trans"], c["N"], c["K"], c["alpha"], A, c["offA"], c["lda"], c["beta"],
                             C, c["offC"], c["ldc"], impl="ref")
            else:
                oracle.csyr2k(c["order"], c["uplo"], c["trans"], c["N"], c["K"], c["alpha"], A, c["offA"], c["lda"], B, c["offB"],
                              c["ldb"], c["beta"], C, c["offC"], c["ldc"], impl="ref")
            out[name] = C
        else:
            out[name] = hermitian_update_by_external_blas(c)
    for name, c in cc.golden_csymm_cases().items():
        out[name] = complex_symm_by_external_blas(c)
    for name, c in cc.golden_ctrmm_cases().items():
        A, B = cc.ctrmm_buffers(c)
        oracle.ctrmm(c["order"], c["side"], c["uplo"], c["transA"], c["diag"], c["M"], c["N"], c["alpha"], A, c["offA"], c["lda"],
                     B, c["offB"], c["ldb"], impl="ref")
        out[name] = B
    path = os.path.join(os.path.dirname(__file__), "level3_golden.npz")
    np.savez_compressed(path, **out)
    print(f"wrote {path}: {len(out)} cases, {os.path.getsize(path)} bytes")


if __name__ == "__main__":
    main()
