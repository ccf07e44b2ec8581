"""Pins the complex GEMM part of the CPU oracle to the reference's NaiveBlas::gemm<FloatComplex/DoubleComplex>
(src/library/tools/ktest/naive/naive_blas.cpp:546-578 with the complex operators at :297-372): committed
golden outputs made with that code, the code itself where it was compiled, exact integers."""
import os

import numpy as np
import pytest

import oracle
from oracle import NoTrans
from tests import cases_complex as cc

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "level3_golden.npz")


def run(c, impl, logical=None):
    A, B, C = cc.cgemm_buffers(c, logical)
    oracle.cgemm(c["order"], c["transA"], c["transB"], c["M"], c["N"], c["K"], c["alpha"], A, c["offA"], c["lda"],
                 B, c["offB"], c["ldb"], c["beta"], C, c["offC"], c["ldc"], impl=impl)
    return C


def same_bits(a, b):
    return a.shape == b.shape and np.array_equal(a.view(np.uint8), b.view(np.uint8))


def test_port_matches_golden(built_oracle):
    g = np.load(GOLDEN)
    items = list(cc.golden_cgemm_cases().items())
    assert len(items) == 36
    for name, c in items:
        assert same_bits(run(c, "port"), g[name]), name


@pytest.mark.skipif(not oracle.have_ref(), reason="reference's own naive_blas.cpp was not compiled here")
def test_port_matches_reference_code(built_oracle):
    for prec in "cz":
        for c in cc.sweep_cgemm_cases(prec, "uniform")[::4]:
            if max(c["M"], c["N"], c["K"]) > 150:
                continue
            assert same_bits(run(c, "port"), run(c, "ref")), c


def test_integer_inputs_are_exact(built_oracle):
    for c in cc.sweep_cgemm_cases("z", "int")[::3]:
        logical = cc.cgemm_logical(c)
        got = oracle.view(run(c, "port", logical), c["order"], NoTrans, c["M"], c["N"], c["ldc"], c["offC"])
        want, _ = cc.cgemm_exact(c, logical)
        assert np.array_equal(got, want), c


# ------------------------------------------------------------------------------------- complex TRSM
def run_trsm(c, impl, logical=None):
    A, B = cc.ctrsm_buffers(c, logical)
    oracle.ctrsm(c["order"], c["side"], c["uplo"], c["transA"], c["diag"], c["M"], c["N"], c["alpha"], A, c["offA"], c["lda"],
                 B, c["offB"], c["ldb"], impl=impl)
    return B


def test_trsm_port_matches_golden(built_oracle):
    """Golden outputs made with NaiveBlas::trsm<FloatComplex/DoubleComplex> (naive_blas.cpp:632-690)."""
    g = np.load(GOLDEN)
    items = list(cc.golden_ctrsm_cases().items())
    assert len(items) == 96
    for name, c in items:
        assert same_bits(run_trsm(c, "port"), g[name]), name


@pytest.mark.skipif(not oracle.have_ref(), reason="reference's own naive_blas.cpp was not compiled here")
def test_trsm_port_matches_reference_code(built_oracle):
    for prec in "cz":
        for c in cc.sweep_ctrsm_cases(prec)[::7]:
            if max(c["M"], c["N"]) > 140:
                continue
            assert same_bits(run_trsm(c, "port"), run_trsm(c, "ref")), c


def test_trsm_solves_the_system(built_oracle):
    """Poisoned entries are never read and the solution satisfies op(A) X = alpha B within the bound."""
    for c in cc.sweep_ctrsm_cases("z")[::5]:
        if max(c["M"], c["N"]) > 140:
            continue
        logical = cc.ctrsm_logical(c)
        X = oracle.view(run_trsm(c, "port", logical), c["order"], NoTrans, c["M"], c["N"], c["ldb"], c["offB"])
        assert np.all(np.isfinite(X)), c
        assert cc.ctrsm_backward_ratio(c, X, cc.ctrsm_op_triangle(c, logical[0]), logical[1]) <= 1.0, c


# ------------------------------------------------------------------------------------- complex TRMM
def run_trmm(c, impl, logical=None):
    A, B = cc.ctrmm_buffers(c, logical)
    oracle.ctrmm(c["order"], c["side"], c["uplo"], c["transA"], c["diag"], c["M"], c["N"], c["alpha"], A, c["offA"], c["lda"],
                 B, c["offB"], c["ldb"], impl=impl)
    return B


def test_trmm_port_matches_golden(built_oracle):
    """Golden outputs made with NaiveBlas::trmm<FloatComplex/DoubleComplex> (naive_blas.cpp:580-630)."""
    g = np.load(GOLDEN)
    items = list(cc.golden_ctrmm_cases().items())
    assert len(items) == 96
    for name, c in items:
        assert same_bits(run_trmm(c, "port"), g[name]), name


@pytest.mark.skipif(not oracle.have_ref(), reason="reference's own naive_blas.cpp was not compiled here")
def test_trmm_port_matches_reference_code(built_oracle):
    for prec in "cz":
        for c in cc.sweep_ctrmm_cases(prec, "uniform")[::7]:
            if max(c["M"], c["N"]) > 140:
                continue
            assert same_bits(run_trmm(c, "port"), run_trmm(c, "ref")), c


def test_trmm_integer_inputs_are_exact_and_poison_is_not_read(built_oracle):
    for c in cc.sweep_ctrmm_cases("z", "int")[::5]:
        if max(c["M"], c["N"]) > 140:
            continue
        logical = cc.ctrmm_logical(c)
        X = oracle.view(run_trmm(c, "port", logical), c["order"], NoTrans, c["M"], c["N"], c["ldb"], c["offB"])
        want, _, _ = cc.ctrmm_exact(c, logical)
        assert np.array_equal(X, want), c
