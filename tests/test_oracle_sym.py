"""Pins the SYR2K and SYMM parts of the CPU oracle.

SYR2K follows the reference's NaiveBlas::syr2k (src/library/tools/ktest/naive/naive_blas.cpp:728-766):
committed golden outputs made with that code, the code itself where it was compiled, exact integers.
SYMM has no counterpart in the reference's naive BLAS: the reference's tests compare with an external
Fortran BLAS (src/tests/correctness/blas-lapack.h), so the golden outputs come from that interface
(OpenBLAS through scipy) and the restatement must equal them on integer inputs and stay within
4*n*u of them on real inputs."""
import os

import numpy as np
import pytest

import oracle
from oracle import Left, NoTrans
from tests import cases, cases_sym

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "level3_golden.npz")


def run_syr2k(c, impl):
    A, B, C = cases_sym.syr2k_buffers(c)
    oracle.syr2k(c["order"], c["uplo"], c["trans"], c["N"], c["K"], c["alpha"], A, c["offA"], c["lda"], B, c["offB"], c["ldb"],
                 c["beta"], C, c["offC"], c["ldc"], impl=impl)
    return C


def run_symm(c, logical=None):
    A, B, C = cases_sym.symm_buffers(c, logical)
    oracle.symm(c["order"], c["side"], c["uplo"], c["M"], c["N"], c["alpha"], A, c["offA"], c["lda"], B, c["offB"], c["ldb"],
                c["beta"], C, c["offC"], c["ldc"])
    return C


def same_bits(a, b):
    return a.shape == b.shape and np.array_equal(a.view(np.uint8), b.view(np.uint8))


def test_syr2k_port_matches_golden(built_oracle):
    g = np.load(GOLDEN)
    names = list(cases_sym.golden_syr2k_cases().items())
    assert len(names) == 16
    for name, c in names:
        assert same_bits(run_syr2k(c, "port"), g[name]), name


@pytest.mark.skipif(not oracle.have_ref(), reason="reference's own naive_blas.cpp was not compiled here")
def test_syr2k_port_matches_reference_code(built_oracle):
    for prec in "sd":
        for c in cases_sym.sweep_syr2k_cases(prec, "uniform")[::5]:
            if c["N"] > 140:
                continue
            assert same_bits(run_syr2k(c, "port"), run_syr2k(c, "ref")), c


def test_syr2k_integer_inputs_are_exact(built_oracle):
    for c in cases_sym.sweep_syr2k_cases("d", "int")[::4]:
        if c["N"] > 140:
            continue
        opA, opB, C = cases_sym.syr2k_logical(c)
        got = oracle.view(run_syr2k(c, "port"), c["order"], NoTrans, c["N"], c["N"], c["ldc"], c["offC"])
        want = c["alpha"] * (opA @ opB.T + opB @ opA.T) + c["beta"] * np.nan_to_num(C)
        tri = ~cases_sym.other_triangle(c["N"], c["uplo"])
        assert np.array_equal(got[tri], want[tri]), c
        assert np.all(np.isnan(got[~tri])), c


def test_symm_port_against_external_blas_golden(built_oracle):
    g = np.load(GOLDEN)
    names = list(cases_sym.golden_symm_cases().items())
    assert len(names) == 16
    for name, c in names:
        got, want = run_symm(c), g[name]
        mask = oracle.outside_mask(got.size, c["order"], NoTrans, c["M"], c["N"], c["ldc"], c["offC"])
        assert same_bits(got[mask], want[mask]), name
        X = oracle.view(got, c["order"], NoTrans, c["M"], c["N"], c["ldc"], c["offC"])
        W = oracle.view(want, c["order"], NoTrans, c["M"], c["N"], c["ldc"], c["offC"])
        if c["mode"] == "int":
            assert np.array_equal(X, W), name
        else:
            _, mag = cases_sym.symm_exact(c, cases_sym.symm_logical(c))
            n = c["M"] if c["side"] == Left else c["N"]
            assert np.all(np.abs(X.astype(np.float64) - W) <= 4 * n * oracle.unit_roundoff(cases.DT[c["prec"]]) * mag), name


def test_symm_integer_inputs_are_exact_and_other_triangle_is_not_read(built_oracle):
    for c in cases_sym.sweep_symm_cases("d", "int")[::3]:
        if max(c["M"], c["N"]) > 300:
            continue
        logical = cases_sym.symm_logical(c)
        got = oracle.view(run_symm(c, logical), c["order"], NoTrans, c["M"], c["N"], c["ldc"], c["offC"])
        want, _ = cases_sym.symm_exact(c, logical)
        assert np.array_equal(got, want), c
