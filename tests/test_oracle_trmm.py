"""Pins the TRMM part of the CPU oracle to the reference's NaiveBlas::trmm
(src/library/tools/ktest/naive/naive_blas.cpp:580-630): committed golden outputs, the reference code
itself where it was compiled, and the exact float64 product."""
import os

import numpy as np
import pytest

import oracle
from oracle import NoTrans
from tests import cases_trmm

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "level3_golden.npz")


def run(c, impl):
    A, B = cases_trmm.trmm_buffers(c)
    oracle.trmm(c["order"], c["side"], c["uplo"], c["transA"], c["diag"], c["M"], c["N"], c["alpha"], A, c["offA"], c["lda"],
                B, c["offB"], c["ldb"], impl=impl)
    return B


def same_bits(a, b):
    return a.shape == b.shape and np.array_equal(a.view(np.uint8), b.view(np.uint8))


def test_port_matches_golden(built_oracle):
    g = np.load(GOLDEN)
    n = 0
    for name, c in cases_trmm.golden_trmm_cases().items():
        assert same_bits(run(c, "port"), g[name]), name
        n += 1
    assert n == 64


@pytest.mark.skipif(not oracle.have_ref(), reason="reference's own naive_blas.cpp was not compiled here")
def test_port_matches_reference_code(built_oracle):
    for prec in "sd":
        for c in cases_trmm.sweep_trmm_cases(prec, "uniform")[::7]:
            if max(c["M"], c["N"]) > 140:
                continue
            assert same_bits(run(c, "port"), run(c, "ref")), c


def test_integer_inputs_are_exact_and_poison_is_not_read(built_oracle):
    for c in cases_trmm.sweep_trmm_cases("d", "int")[::5]:
        if max(c["M"], c["N"]) > 140:
            continue
        A, B = cases_trmm.trmm_logical(c)
        got = run(c, "port")
        X = oracle.view(got, c["order"], NoTrans, c["M"], c["N"], c["ldb"], c["offB"])
        want, _ = cases_trmm.trmm_exact(c, A, B)
        assert np.array_equal(X, want), c
