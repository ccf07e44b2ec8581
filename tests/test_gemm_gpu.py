"""GEMM parity on the GPU, through the C ABI, against the CPU oracle.

Mirrors the reference's correctness strategy (src/tests/correctness/corr-gemm.cpp:50-206):
integer-valued inputs whose partial sums are all exactly representable must reproduce the oracle
BIT FOR BIT (the reference asserts |ref - got| <= 0, src/tests/include/matrix.h:301-329); real-valued
inputs must meet max |C - C_exact| / (|alpha| |A||B| + |beta||C|) <= 4*K*u (u = 2^-24 / 2^-53).
Every element outside the output matrix (offset head, leading-dimension padding, tail) is NaN
before the call and must keep its bits."""
import numpy as np
import pytest
import torch

import oracle
from oracle import ColumnMajor, NoTrans, RowMajor, Trans
from tests import cases
from tests.gpu_util import outside_untouched, run_gemm_gpu, run_gemm_oracle, same_bits

pytestmark = pytest.mark.gpu


def check_real(cb, c, forced_path=None):
    logical = cases.gemm_logical(c)
    bufs = cases.gemm_buffers(c, logical)
    before = bufs[2].copy()
    st, got = run_gemm_gpu(cb, c, bufs)
    assert st == cb.clblasSuccess, (cb.STATUS_NAME.get(st, st), c)
    assert outside_untouched(before, got, c), c
    Cg = oracle.view(got, c["order"], NoTrans, c["M"], c["N"], c["ldc"], c["offC"])
    assert np.all(np.isfinite(Cg)), c
    opA, opB, C = logical
    ratio = oracle.gemm_error_ratio(Cg, c["alpha"], opA, opB, c["beta"], C, c["K"], cases.DT[c["prec"]])
    assert ratio <= 1.0, (ratio, c)
    return ratio


def check_exact(cb, c):
    bufs = cases.gemm_buffers(c)
    st, got = run_gemm_gpu(cb, c, bufs)
    assert st == cb.clblasSuccess, (cb.STATUS_NAME.get(st, st), c)
    want = run_gemm_oracle(c, bufs)
    assert same_bits(got, want), c


@pytest.mark.parametrize("prec", ["s", "d"])
@pytest.mark.parametrize("path", [0, 1])
def test_sweep_exact_integer(lib, prec, path):
    """Reference-style exact-integer inputs: bit-identical to the oracle, on the automatic dispatch
    and with the alignment-free loader forced."""
    old = lib.set_gemm_path(path)
    try:
        for c in cases.sweep_gemm_cases(prec, "int"):
            check_exact(lib, c)
    finally:
        lib.set_gemm_path(old)


@pytest.mark.parametrize("prec", ["s", "d"])
@pytest.mark.parametrize("path", [0, 1])
def test_sweep_real_valued(lib, prec, path):
    old = lib.set_gemm_path(path)
    try:
        worst = 0.0
        for c in cases.sweep_gemm_cases(prec, "uniform"):
            worst = max(worst, check_real(lib, c))
        assert worst <= 1.0
    finally:
        lib.set_gemm_path(old)


@pytest.mark.parametrize("prec", ["s", "d"])
def test_tile_boundaries(lib, prec):
    """Sizes straddling every tile edge of the kernels (64, 128, 256 +-1) with K ragged as well."""
    seed = 9000
    for ta in (NoTrans, Trans):
        for tb in (NoTrans, Trans):
            for M, N, K in ((127, 129, 31), (128, 128, 32), (129, 127, 33), (255, 257, 17), (257, 255, 64),
                            (384, 130, 100), (1, 300, 5), (300, 1, 7), (513, 65, 1)):
                seed += 1
                check_exact(lib, cases.gemm_case(prec, ColumnMajor, ta, tb, M, N, K, alpha=1.0, beta=2.0,
                                                 mode="int", seed=seed))
                # aligned leading dimensions with ragged sizes (the TMA paths' out-of-bounds fill)
                check_exact(lib, cases.gemm_case(prec, ColumnMajor, ta, tb, M, N, K, alpha=3.0, beta=0.0,
                                                 pad=(8 - M % 8 if not ta else 8 - K % 8, 4, 4), mode="int", seed=seed))


@pytest.mark.parametrize("prec", ["s", "d"])
def test_beta_zero_never_reads_c(lib, prec):
    """beta == 0: C is an output only; NaN in it must not reach the result (the reference selects a
    separate kernel that never loads C, src/library/blas/AutoGemm/KernelOpenCL.py:100-104)."""
    for M, N, K in ((64, 64, 64), (130, 70, 33), (512, 384, 256)):
        c = cases.gemm_case(prec, ColumnMajor, NoTrans, Trans, M, N, K, alpha=1.0, beta=0.0, mode="int")
        opA, opB, C = cases.gemm_logical(c)
        C[...] = np.nan
        bufs = cases.gemm_buffers(c, (opA, opB, C))
        st, got = run_gemm_gpu(lib, c, bufs)
        assert st == lib.clblasSuccess
        Cg = oracle.view(got, ColumnMajor, NoTrans, M, N, c["ldc"], 0)
        assert np.array_equal(Cg, (opA.astype(np.float64) @ opB.astype(np.float64)).astype(cases.DT[prec]))


@pytest.mark.parametrize("prec", ["s", "d"])
def test_k_zero_and_alpha_zero(lib, prec):
    """K == 0 skips the A/B checks and means C <- beta*C (src/library/blas/xgemm.cc:691); alpha == 0
    is the same operation and must not read A or B (they are all NaN here)."""
    c = cases.gemm_case(prec, ColumnMajor, NoTrans, NoTrans, 37, 21, 0, alpha=1.0, beta=-2.0, pad=(0, 0, 3))
    dt = cases.DT[prec]
    C = oracle.uniform((37, 21), dt, 5, 1)
    Cb = oracle.pack(C, ColumnMajor, NoTrans, c["ldc"], 0)
    A = np.full(4, np.nan, dtype=dt)
    st, got = run_gemm_gpu(lib, c, (A, A, Cb))
    assert st == lib.clblasSuccess
    assert np.array_equal(oracle.view(got, ColumnMajor, NoTrans, 37, 21, c["ldc"], 0), (-2.0 * C).astype(dt))
    assert outside_untouched(Cb, got, c)

    c = cases.gemm_case(prec, RowMajor, Trans, NoTrans, 33, 65, 17, alpha=0.0, beta=0.5)
    opA, opB, C = cases.gemm_logical(c)
    bufs = cases.gemm_buffers(c, (opA * np.nan, opB * np.nan, C))
    st, got = run_gemm_gpu(lib, c, bufs)
    assert st == lib.clblasSuccess
    assert np.array_equal(oracle.view(got, RowMajor, NoTrans, 33, 65, c["ldc"], 0), (0.5 * C).astype(dt))


def test_config1_sgemm_1024(lib):
    """SGEMM column-major N/N 1024^3, U[-1,1], alpha 1.5, beta 0.5: checked entry by entry against the
    oracle-grade float64 product with the 4*K*u bound, and bit for bit on integer inputs."""
    c = cases.gemm_case("s", ColumnMajor, NoTrans, NoTrans, 1024, 1024, 1024, alpha=1.5, beta=0.5)
    check_real(lib, c)
    assert lib.last_gemm_kernel() != "none"
    ci = cases.gemm_case("s", ColumnMajor, NoTrans, NoTrans, 1024, 1024, 1024, alpha=2.0, beta=3.0, mode="int")
    bufs = cases.gemm_buffers(ci)
    st, got = run_gemm_gpu(lib, ci, bufs)
    opA, opB, C = cases.gemm_logical(ci)
    want = (2.0 * (opA.astype(np.float64) @ opB.astype(np.float64)) + 3.0 * C).astype(np.float32)
    assert st == lib.clblasSuccess
    assert np.array_equal(oracle.view(got, ColumnMajor, NoTrans, 1024, 1024, 1024, 0), want)


def test_config3_sgemm_rowmajor_ragged(lib):
    """SGEMM row-major T/N, M=4099 N=3001 K=1537, lda=M+16, ldb=N+32, ldc=N+8, offsets 7/13/5,
    alpha=-2, beta=0.25: unaligned bases and odd leading dimensions, ragged M, N and K."""
    c = cases.gemm_case("s", RowMajor, Trans, NoTrans, 4099, 3001, 1537, alpha=-2.0, beta=0.25,
                        pad=(16, 32, 8), off=(7, 13, 5))
    assert (c["lda"], c["ldb"], c["ldc"]) == (4099 + 16, 3001 + 32, 3001 + 8)
    # automatic dispatch: operands are copied once into an aligned workspace, then the TMA kernel runs
    check_real(lib, c)
    assert lib.last_gemm_kernel() == "sgemm_ffma_tma"
    # the alignment-free kernel on the same problem, in place
    old = lib.set_gemm_path(1)
    try:
        check_real(lib, c)
        assert lib.last_gemm_kernel() == "gemm_simt_ldg"
        ci = cases.gemm_case("s", RowMajor, Trans, NoTrans, 4099, 3001, 1537, alpha=-2.0, beta=3.0,
                             pad=(16, 32, 8), off=(7, 13, 5), mode="int")
        bufs = cases.gemm_buffers(ci)
        st, got_simt = run_gemm_gpu(lib, ci, bufs)
        assert st == lib.clblasSuccess
    finally:
        lib.set_gemm_path(old)
    # integer-valued inputs: both routes give the same bits, padding and offsets untouched
    st, got_auto = run_gemm_gpu(lib, ci, bufs)
    assert st == lib.clblasSuccess and same_bits(got_auto, got_simt)
    assert outside_untouched(bufs[2], got_auto, ci)


def _aligned_case(prec, order, ta, tb, M, N, K, seed, mode="int", alpha=2.0, beta=3.0):
    """Leading dimensions rounded up to 16 bytes and zero offsets: what the TMA paths accept."""
    q = 4 if prec == "s" else 2
    c = cases.gemm_case(prec, order, ta, tb, M, N, K, alpha=alpha, beta=beta, mode=mode, seed=seed)
    for k in ("lda", "ldb", "ldc"):
        c[k] = (c[k] + q - 1) // q * q
    return c


@pytest.mark.parametrize("prec,kernel", [("s", "sgemm_ffma_tma"), ("d", "dgemm_mma_tma")])
def test_tma_paths_exact(lib, prec, kernel):
    """TMA-staged kernels, all four transposes and both orders, sizes straddling the 128 tile and the
    K slab, ragged M, N, K served by TMA's out-of-bounds zero fill: bit-identical to the oracle."""
    seed = 20000
    for order in (ColumnMajor, RowMajor):
        for ta in (NoTrans, Trans):
            for tb in (NoTrans, Trans):
                for M, N, K in ((128, 128, 32), (256, 128, 64), (127, 129, 33), (130, 250, 17), (1, 1, 1), (64, 300, 100),
                                (384, 257, 161), (5, 3, 200)):
                    seed += 1
                    check_exact(lib, _aligned_case(prec, order, ta, tb, M, N, K, seed))
                    assert lib.last_gemm_kernel() == kernel
                    check_exact(lib, _aligned_case(prec, order, ta, tb, M, N, K, seed, beta=0.0))
    assert lib.device_fault() == 0


@pytest.mark.parametrize("prec", ["s", "d"])
def test_tma_paths_real_valued(lib, prec):
    seed = 21000
    for ta in (NoTrans, Trans):
        for tb in (NoTrans, Trans):
            for M, N, K in ((512, 384, 1000), (257, 129, 2049)):
                seed += 1
                check_real(lib, _aligned_case(prec, ColumnMajor, ta, tb, M, N, K, seed, mode="uniform", alpha=1.5, beta=0.5))
                assert lib.last_gemm_kernel().endswith("_tma")
    assert lib.device_fault() == 0


def test_sgemm_split_k_exact(lib):
    """Few tiles and a long K: the SGEMM path splits K over several CTAs per tile (partial tiles in a workspace, ordered
    reduction).  Integer inputs must still equal the oracle, for all transposes, ragged sizes and beta = 0."""
    seed = 22000
    for ta in (NoTrans, Trans):
        for tb in (NoTrans, Trans):
            for M, N, K in ((512, 512, 512), (768, 300, 2048), (130, 257, 1100), (64, 64, 4097)):
                seed += 1
                check_exact(lib, _aligned_case("s", ColumnMajor, ta, tb, M, N, K, seed))
                assert lib.last_gemm_kernel() == "sgemm_ffma_tma"
                check_exact(lib, _aligned_case("s", RowMajor, ta, tb, M, N, K, seed, beta=0.0))
    assert lib.device_fault() == 0


def test_dgemm_stream_k_tail_exact(lib):
    """More than one wave of tiles and a partial last wave: the DGEMM path gives the last tiles to the kernel that shares
    their K range between CTAs (partial tiles in a workspace, the last arrival sums them in slot order).  Integer inputs
    must equal the oracle for all transposes, ragged edges included, and twice the same call must agree bit for bit."""
    seed = 23000
    for ta in (NoTrans, Trans):
        for tb in (NoTrans, Trans):
            for M, N, K in ((2048, 2048, 512), (1990, 2300, 700), (1280, 3000, 1030), (2560, 1920, 256)):
                seed += 1
                check_exact(lib, _aligned_case("d", ColumnMajor, ta, tb, M, N, K, seed))
                assert lib.last_gemm_kernel() == "dgemm_mma_tma"
    check_exact(lib, _aligned_case("d", RowMajor, Trans, NoTrans, 2100, 2100, 900, 23099, beta=0.0))
    c = _aligned_case("d", ColumnMajor, NoTrans, Trans, 2304, 2176, 1111, 23100, mode="uniform", alpha=1.5, beta=0.5)
    bufs = cases.gemm_buffers(c)
    _, first = run_gemm_gpu(lib, c, bufs)
    _, second = run_gemm_gpu(lib, c, bufs)
    assert same_bits(first, second)
    assert lib.device_fault() == 0


def test_config2_shape_family_dgemm_tn(lib):
    """DGEMM column-major T/N, normal(0,1), alpha = beta = 1, tight leading dimensions (the benchmark's
    DGEMM workload) at 1024^3, where the float64 host check is cheap; the 8192^3 run is checked through
    sampled rows/columns in test_full_configs_gpu.py."""
    c = cases.gemm_case("d", ColumnMajor, Trans, NoTrans, 1024, 1024, 1024, alpha=1.0, beta=1.0, mode="normal")
    r = check_real(lib, c)
    assert lib.last_gemm_kernel() == "dgemm_mma_tma"
    assert r <= 1.0


@pytest.mark.parametrize("prec", ["s", "d"])
def test_repacked_operands_exact(lib, prec):
    """Large products whose operands TMA cannot address (odd leading dimensions, offset bases) or, for
    SGEMM, whose operands are K-contiguous: the dispatcher copies / transposes them into an aligned
    workspace first.  Integer-valued inputs, compared bit for bit with the exact float64 product."""
    dt = cases.DT[prec]
    seed = 30000
    for order in (ColumnMajor, RowMajor):
        for ta in (NoTrans, Trans):
            for tb in (NoTrans, Trans):
                seed += 1
                M, N, K = 2049, 2111, 2053
                c = cases.gemm_case(prec, order, ta, tb, M, N, K, alpha=2.0, beta=-1.0, pad=(3, 5, 1), off=(1, 2, 3),
                                    mode="int", seed=seed)
                opA, opB, C = cases.gemm_logical(c)
                bufs = cases.gemm_buffers(c, (opA, opB, C))
                st, got = run_gemm_gpu(lib, c, bufs)
                assert st == lib.clblasSuccess
                assert lib.last_gemm_kernel().endswith("_tma"), lib.last_gemm_kernel()
                want = (2.0 * (opA.astype(np.float64) @ opB.astype(np.float64)) - C.astype(np.float64)).astype(dt)
                assert np.array_equal(oracle.view(got, order, NoTrans, M, N, c["ldc"], c["offC"]), want), c
                assert outside_untouched(bufs[2], got, c)
    assert lib.device_fault() == 0


def test_sgemm_transposed_in_16_byte_accesses_exact(lib):
    """Aligned K-contiguous SGEMM operands of a product large enough to be transposed first (the 16-byte path of the
    transposition kernel, edges that are not multiples of its 64 x 64 tile): every transposition ends in the N/T
    kernel and must give the exact product of the integer-valued inputs."""
    seed = 31000
    for order in (ColumnMajor, RowMajor):
        for ta, tb in ((NoTrans, NoTrans), (Trans, NoTrans), (Trans, Trans)):
            seed += 1
            M, N, K = 2052, 2116, 2056
            c = cases.gemm_case("s", order, ta, tb, M, N, K, alpha=1.0, beta=2.0, mode="int", seed=seed)
            opA, opB, C = cases.gemm_logical(c)
            bufs = cases.gemm_buffers(c, (opA, opB, C), tail=0)
            st, got = run_gemm_gpu(lib, c, bufs)
            assert st == lib.clblasSuccess
            assert "<N,T," in lib.last_gemm_variant() or lib.last_gemm_variant().startswith("sgemm_nt_16x8"), lib.last_gemm_variant()
            want = (opA.astype(np.float64) @ opB.astype(np.float64) + 2.0 * C.astype(np.float64)).astype(np.float32)
            assert np.array_equal(oracle.view(got, order, NoTrans, M, N, c["ldc"], c["offC"]), want), c
    assert lib.device_fault() == 0
