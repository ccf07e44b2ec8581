"""Pins the complex SYRK / HERK / SYR2K / HER2K / SYMM / HEMM parts of the CPU oracle.

SYRK and SYR2K follow the reference's NaiveBlas::syrk / syr2k on FloatComplex / DoubleComplex
(src/library/tools/ktest/naive/naive_blas.cpp:692-766): golden buffers made with that code, bit for bit.
HERK, HER2K, SYMM and HEMM have no counterpart there (the reference's tests call an external Fortran BLAS,
src/tests/correctness/blas-lapack.h): their golden results come from that interface (OpenBLAS through scipy)
and the restatement must equal them on integer inputs and stay within 4*k*u on real ones."""
import os

import numpy as np
import pytest

import oracle
from oracle import Left, NoTrans
from tests import cases_complex as cc

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "level3_golden.npz")


def run_rank(c, impl="port", logical=None):
    A, B, C = cc.crank_buffers(c, logical)
    herm = c["kind"] in ("herk", "her2k")
    if c["kind"] in ("syrk", "herk"):
        oracle.csyrk(c["order"], c["uplo"], c["trans"], c["N"], c["K"], c["alpha"], A, c["offA"], c["lda"], c["beta"], C, c["offC"],
                     c["ldc"], herm=herm, impl=impl)
    else:
        oracle.csyr2k(c["order"], c["uplo"], c["trans"], c["N"], c["K"], c["alpha"], A, c["offA"], c["lda"], B, c["offB"], c["ldb"],
                      c["beta"], C, c["offC"], c["ldc"], herm=herm, impl=impl)
    return C


def run_symm(c, logical=None):
    A, B, C = cc.csymm_buffers(c, logical)
    oracle.csymm(c["order"], c["side"], c["uplo"], c["M"], c["N"], c["alpha"], A, c["offA"], c["lda"], B, c["offB"], c["ldb"],
                 c["beta"], C, c["offC"], c["ldc"], herm=c["kind"] == "hemm")
    return C


def same_bits(a, b):
    return a.shape == b.shape and np.array_equal(a.view(np.uint8), b.view(np.uint8))


def test_rank_updates_against_golden(built_oracle):
    g = np.load(GOLDEN)
    items = list(cc.golden_crank_cases().items())
    assert len(items) == 64
    for name, c in items:
        got = run_rank(c)
        if c["kind"] in ("syrk", "syr2k"):
            assert same_bits(got, g[name]), name                     # made with the reference's own code
            continue
        X = oracle.view(got, c["order"], NoTrans, c["N"], c["N"], c["ldc"], c["offC"])
        W = g[name]
        tri = ~cc._other_triangle(c["N"], c["uplo"])
        assert np.all(np.isnan(X[~tri])), name
        if c["mode"] == "int":
            assert np.array_equal(X[tri], W[tri]), name
        else:
            _, mag = cc.crank_exact(c, cc.crank_logical(c))
            k = c["K"] * (4 if c["kind"] == "her2k" else 2)
            assert np.all(np.abs(X.astype(np.complex128) - W)[tri] <= (4 * k * oracle.unit_roundoff(cc.RDT[c["prec"]]) * mag)[tri]), name


@pytest.mark.skipif(not oracle.have_ref(), reason="reference's own naive_blas.cpp was not compiled here")
def test_symmetric_updates_match_reference_code(built_oracle):
    for kind in ("syrk", "syr2k"):
        for prec in "cz":
            for c in cc.sweep_crank_cases(kind, prec, "uniform")[::3]:
                if c["N"] > 140:
                    continue
                assert same_bits(run_rank(c, "port"), run_rank(c, "ref")), c


def test_rank_updates_exact_on_integers(built_oracle):
    for kind in ("syrk", "herk", "syr2k", "her2k"):
        for c in cc.sweep_crank_cases(kind, "z", "int")[::3]:
            if c["N"] > 140:
                continue
            logical = cc.crank_logical(c)
            X = oracle.view(run_rank(c, "port", logical), c["order"], NoTrans, c["N"], c["N"], c["ldc"], c["offC"])
            want, _ = cc.crank_exact(c, logical)
            tri = ~cc._other_triangle(c["N"], c["uplo"])
            assert np.array_equal(X[tri], want[tri]), c
            assert np.all(np.isnan(X[~tri])), c


def test_symm_hemm_against_external_blas_golden(built_oracle):
    g = np.load(GOLDEN)
    items = list(cc.golden_csymm_cases().items())
    assert len(items) == 32
    for name, c in items:
        X = oracle.view(run_symm(c), c["order"], NoTrans, c["M"], c["N"], c["ldc"], c["offC"])
        W = g[name]
        if c["mode"] == "int":
            assert np.array_equal(X, W), name
        else:
            _, mag = cc.csymm_exact(c, cc.csymm_logical(c))
            n = c["M"] if c["side"] == Left else c["N"]
            assert np.all(np.abs(X.astype(np.complex128) - W) <= 4 * 2 * n * oracle.unit_roundoff(cc.RDT[c["prec"]]) * mag), name


def test_symm_hemm_exact_on_integers(built_oracle):
    for kind in ("symm", "hemm"):
        for c in cc.sweep_csymm_cases(kind, "z", "int")[::3]:
            logical = cc.csymm_logical(c)
            X = oracle.view(run_symm(c, logical), c["order"], NoTrans, c["M"], c["N"], c["ldc"], c["offC"])
            want, _ = cc.csymm_exact(c, logical)
            assert np.array_equal(X, want), c
