"""Pins the SYRK part of the CPU oracle to the reference's NaiveBlas::syrk
(src/library/tools/ktest/naive/naive_blas.cpp:692-727): committed golden outputs, the reference code
itself where it was compiled, and the exact float64 product on integer inputs."""
import os

import numpy as np
import pytest

import oracle
from oracle import Lower, NoTrans
from tests import cases_syrk

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "level3_golden.npz")


def run(c, impl):
    A, C = cases_syrk.syrk_buffers(c)
    oracle.syrk(c["order"], c["uplo"], c["trans"], c["N"], c["K"], c["alpha"], A, c["offA"], c["lda"], c["beta"], C,
                c["offC"], c["ldc"], impl=impl)
    return C


def same_bits(a, b):
    return a.shape == b.shape and np.array_equal(a.view(np.uint8), b.view(np.uint8))


def test_port_matches_golden(built_oracle):
    g = np.load(GOLDEN)
    n = 0
    for name, c in cases_syrk.golden_syrk_cases().items():
        assert same_bits(run(c, "port"), g[name]), name
        n += 1
    assert n == 16


@pytest.mark.skipif(not oracle.have_ref(), reason="reference's own naive_blas.cpp was not compiled here")
def test_port_matches_reference_code(built_oracle):
    for prec in "sd":
        for c in cases_syrk.sweep_syrk_cases(prec, "uniform")[::5]:
            if c["N"] > 140:
                continue
            assert same_bits(run(c, "port"), run(c, "ref")), c


def test_integer_inputs_are_exact_and_other_triangle_is_kept(built_oracle):
    for c in cases_syrk.sweep_syrk_cases("d", "int")[::4]:
        if c["N"] > 140:
            continue
        opA, C = cases_syrk.syrk_logical(c)
        got = oracle.view(run(c, "port"), c["order"], NoTrans, c["N"], c["N"], c["ldc"], c["offC"])
        want = c["alpha"] * (opA @ opA.T) + c["beta"] * np.nan_to_num(C)
        tri = np.tril(np.ones_like(C, dtype=bool)) if c["uplo"] == Lower else np.triu(np.ones_like(C, dtype=bool))
        assert np.array_equal(got[tri], want[tri]), c
        assert np.all(np.isnan(got[~tri])), c
