"""The reference suite's large cases and one test per kernel instantiation, through the C ABI.

* TRSM over order x side x uplo x trans x diag at order 1100 (nine 128-blocks, odd splits at every level of the
  recursion) and one pass at the reference's "Big" size 2801 x 2903
  (src/tests/correctness/test-correctness.cpp:831-853, :994-1016); accepted by the backward-error bound AND by the
  reference's own element-wise rule (trsmDelta, src/tests/correctness/trsm-delta.h:44-240) against the oracle.
* GEMM "SelectedBig" shapes 5777 x 5333 x 3000 T/N and 6777 x 3333 x 3000 T/ConjTrans (:675-700), integer-valued
  inputs whose partial sums are exact, so any correct summation order gives the same bits: the expected result is a
  float64 host product of the same integers.
* Products sized so that each variant of the kernels is the one that runs -- asserted through
  clblasB200LastGemmVariant -- the 16 x 8 register-tile SGEMM and its triangular instantiation (SSYRK, CHERK),
  the DGEMM stream-K tail, SGEMM split-K.
* Several command queues on one device (the reference's MultipleQueues cases, :3006-3042: sizes 513 and 1025).
* A conditioning sweep of the inverse-based TRSM.
"""
import itertools

import numpy as np
import pytest
import torch

import oracle
from oracle import ColumnMajor, ConjTrans, Left, Lower, NonUnit, NoTrans, Right, RowMajor, Trans, Unit, Upper
from tests import cases
from tests.gpu_util import dev, outside_untouched, run_gemm_gpu, run_trsm_gpu, run_trsm_oracle

pytestmark = pytest.mark.gpu


def _check_trsm(cb, c, with_oracle=True):
    logical = cases.trsm_logical(c)
    bufs = cases.trsm_buffers(c, logical)
    st, got = run_trsm_gpu(cb, c, bufs)
    assert st == cb.clblasSuccess, (cb.STATUS_NAME.get(st, st), c)
    assert outside_untouched(bufs[1], got, c), c
    dt = cases.DT[c["prec"]]
    X = oracle.view(got, c["order"], NoTrans, c["M"], c["N"], c["ldb"], c["offB"])
    assert np.all(np.isfinite(X)), c
    A, B = logical
    T = cases.trsm_op_triangle(c, A)
    ratio = oracle.trsm_backward_ratio(X, c["alpha"], T, B, c["side"], dt)
    assert ratio <= 1.0, (ratio, c)
    if with_oracle:
        want = run_trsm_oracle(c, bufs)
        Xo = oracle.view(want, c["order"], NoTrans, c["M"], c["N"], c["ldb"], c["offB"])
        delta = oracle.trsm_delta(c["side"], c["uplo"], c["transA"], c["diag"], oracle.clean_triangle(A, c["uplo"], c["diag"]),
                                  B, c["alpha"], dt)
        worst = float(np.max(np.abs(X.astype(np.float64) - Xo.astype(np.float64)) / delta))
        assert worst <= 1.0, (worst, c)            # the reference's own acceptance rule


@pytest.mark.parametrize("prec", ["s", "d"])
def test_trsm_order_1100_all_variants(lib, prec):
    seed = 7000
    for order, side, uplo, ta, diag in itertools.product((ColumnMajor, RowMajor), (Left, Right), (Upper, Lower),
                                                         (NoTrans, Trans, ConjTrans), (Unit, NonUnit)):
        seed += 1
        M, N = (1100, 200) if side == Left else (200, 1100)
        _check_trsm(lib, cases.trsm_case(prec, order, side, uplo, ta, diag, M, N, alpha=[1.0, 2.5, -0.5][seed % 3],
                                         pad=(seed % 5, seed % 7), off=(seed % 3, seed % 11), seed=seed))
    assert lib.device_fault() == 0


@pytest.mark.parametrize("prec,order,side,uplo,ta", [("d", ColumnMajor, Left, Lower, NoTrans), ("s", RowMajor, Right, Upper, Trans)])
def test_trsm_reference_big_size(lib, prec, order, side, uplo, ta):
    _check_trsm(lib, cases.trsm_case(prec, order, side, uplo, ta, NonUnit, 2801, 2903, alpha=1.5, seed=7100), with_oracle=False)


def _exact_gemm(cb, prec, order, ta, tb, M, N, K, alpha=2.0, beta=3.0, pad=(0, 0, 0), off=(0, 0, 0), seed=8000, queues=None):
    """Integer-valued inputs (bounds of the reference's generator, src/tests/include/blas-random.h:29-94): the
    device result must equal the float64 host product of the same integers bit for bit."""
    c = cases.gemm_case(prec, order, ta, tb, M, N, K, alpha=alpha, beta=beta, pad=pad, off=off, mode="int", seed=seed)
    opA, opB, C = cases.gemm_logical(c)
    bufs = cases.gemm_buffers(c, (opA, opB, C))
    if queues is None:
        st, got = run_gemm_gpu(cb, c, bufs)
    else:
        dA, dB, dC = (dev(b) for b in bufs)
        fn = cb.clblasSgemm if prec == "s" else cb.clblasDgemm
        events = [torch.cuda.Event() for _ in queues]
        for e, q in zip(events, queues):
            e.record(q)
        torch.cuda.synchronize()
        st = fn(c["order"], c["transA"], c["transB"], M, N, K, alpha, dA, c["offA"], c["lda"], dB, c["offB"], c["ldb"], beta,
                dC, c["offC"], c["ldc"], queues=queues, events=events)
        for e in events:
            e.synchronize()                        # the caller's only way to know: every queue's event
        got = dC.cpu().numpy()
    assert st == cb.clblasSuccess, cb.STATUS_NAME.get(st, st)
    exact = alpha * (opA.astype(np.float64) @ opB.astype(np.float64)) + beta * C.astype(np.float64)
    want = oracle.pack(exact.astype(cases.DT[prec]), order, NoTrans, c["ldc"], c["offC"], tail=3)
    assert outside_untouched(bufs[2], got, c), c
    mask = ~oracle.outside_mask(got.size, order, NoTrans, M, N, c["ldc"], c["offC"])
    # equal as numbers: where the exact result is zero its sign depends on the order of two exact operations
    # (alpha * 0 against beta * c + alpha * 0), which is not part of the reference's rule either (it compares values)
    assert np.array_equal(got[mask], want[mask]), (c, float(np.max(np.abs(got[mask] - want[mask]))))
    return cb.last_gemm_variant()


@pytest.mark.parametrize("order", [ColumnMajor, RowMajor])
def test_gemm_reference_big_shapes(lib, order):
    _exact_gemm(lib, "d", order, Trans, NoTrans, 5777, 5333, 3000, seed=8001)
    _exact_gemm(lib, "s", order, Trans, ConjTrans, 6777, 3333, 3000, seed=8002)
    _exact_gemm(lib, "d", order, NoTrans, NoTrans, 2801, 2903, 3005, seed=8003)
    assert lib.device_fault() == 0


def test_sgemm_16x8_register_tile_kernel_is_exact(lib):
    v = _exact_gemm(lib, "s", ColumnMajor, NoTrans, Trans, 5504, 5504, 1024, seed=8010)          # 1849 tiles: more than 12 per SM
    assert v == "sgemm_nt_16x8", v
    v = _exact_gemm(lib, "s", ColumnMajor, NoTrans, Trans, 5504 - 37, 5504 + 5, 1024 + 19, alpha=-1.0, beta=0.0, seed=8011)
    assert v == "sgemm_nt_16x8", v               # ragged edges in M, N and K


def test_sgemm_split_k_against_wave_quantisation_is_exact(lib):
    """784 tiles of 128 x 128 are 2.65 rounds of CTAs and K = 704 is short: the dispatcher cuts K in two so that the rounds
    come out even.  Same bits as the unsplit product (integer inputs), the same call twice gives the same bits (fixed
    reduction order)."""
    v = _exact_gemm(lib, "s", ColumnMajor, NoTrans, Trans, 3584, 3584, 704, seed=8012)
    assert v == "sgemm_ffma_tma<N,T,128,3,2>+splitk2", v
    import oracle as _o
    g = _o.rng(8013, 0)
    n, k = 3584, 704
    A, B = (torch.from_numpy(g.standard_normal(n * k).astype(np.float32)).cuda() for _ in range(2))
    C1, C2 = torch.zeros(n * n, device="cuda"), torch.zeros(n * n, device="cuda")
    for C in (C1, C2):
        assert lib.clblasSgemm(ColumnMajor, NoTrans, Trans, n, n, k, 1.0, A, 0, n, B, 0, n, 0.0, C, 0, n) == lib.clblasSuccess
    torch.cuda.synchronize()
    assert lib.last_gemm_variant().endswith("+splitk2") and torch.equal(C1, C2)


def test_sgemm_stream_k_is_exact_and_deterministic(lib):
    """Products of about one round of CTAs go to the stream-K kernel (every CTA the same number of K slabs, partial
    tiles added in slot order by the CTA that finishes a tile last): exact on integer inputs, ragged edges included,
    for M-contiguous and K-contiguous A, and bit-identical when repeated."""
    v = _exact_gemm(lib, "s", ColumnMajor, NoTrans, Trans, 1408, 1408, 704, seed=8040)
    assert v == "sgemm_streamk<N,T>", v
    v = _exact_gemm(lib, "s", ColumnMajor, NoTrans, Trans, 1397, 1401, 1100, alpha=-1.0, beta=0.0, pad=(3, 3, 0), seed=8041)      # 11 x 11 tiles
    assert v == "sgemm_streamk<N,T>", v
    v = _exact_gemm(lib, "s", ColumnMajor, Trans, NoTrans, 1408, 1408, 992, seed=8042)           # K-contiguous A: one CTA per SM
    assert v == "sgemm_streamk<T,N>", v
    g = oracle.rng(8043, 0)
    n, k = 1408, 704
    A, B = (torch.from_numpy(g.standard_normal(n * k).astype(np.float32)).cuda() for _ in range(2))
    C1, C2 = torch.zeros(n * n, device="cuda"), torch.zeros(n * n, device="cuda")
    for C in (C1, C2):
        assert lib.clblasSgemm(ColumnMajor, NoTrans, Trans, n, n, k, 1.0, A, 0, n, B, 0, n, 0.0, C, 0, n) == lib.clblasSuccess
    torch.cuda.synchronize()
    assert lib.last_gemm_variant() == "sgemm_streamk<N,T>" and torch.equal(C1, C2)


def test_sgemm_eight_warp_16x8_stream_k_is_exact_and_deterministic(lib):
    """N/T products with a K loop of 36 slabs or more and up to sixteen tiles per SM: one eight-warp CTA per SM, the two
    warp groups take half of every K slab each and swap halves of the tile at the end of a segment; partial tiles are
    added in slot order.  Exact on integer inputs (ragged edges, beta != 0, few tiles with a long K loop, a row-major
    call that maps onto it) and bit-identical when repeated."""
    name = "sgemm_nt_16x8w_streamk"
    assert _exact_gemm(lib, "s", ColumnMajor, NoTrans, Trans, 1280, 1280, 1280, seed=8050) == name
    assert _exact_gemm(lib, "s", ColumnMajor, NoTrans, Trans, 1397, 1401, 1413, alpha=-1.0, beta=0.0, pad=(3, 3, 3), seed=8051) == name
    # a C that does not allow 16-byte accesses stays with the two-CTAs-per-SM kernels
    assert _exact_gemm(lib, "s", ColumnMajor, NoTrans, Trans, 1397, 1401, 1413, pad=(3, 3, 0), seed=8056) != name
    assert _exact_gemm(lib, "s", RowMajor, Trans, NoTrans, 2200, 2056, 1153, seed=8052) == name
    assert _exact_gemm(lib, "s", ColumnMajor, NoTrans, Trans, 300, 200, 8000, seed=8053) == name             # six tiles, 250 slabs
    assert _exact_gemm(lib, "s", ColumnMajor, NoTrans, Trans, 3584, 3584, 1536, seed=8054) == name           # 784 tiles
    assert _exact_gemm(lib, "s", ColumnMajor, NoTrans, Trans, 2048, 2048, 1024, seed=8057) == name           # 32 slabs, uneven rounds
    g = oracle.rng(8055, 0)
    n, k = 2048, 1536
    A, B = (torch.from_numpy(g.standard_normal(n * k).astype(np.float32)).cuda() for _ in range(2))
    C1, C2 = torch.zeros(n * n, device="cuda"), torch.zeros(n * n, device="cuda")
    for C in (C1, C2):
        assert lib.clblasSgemm(ColumnMajor, NoTrans, Trans, n, n, k, 1.0, A, 0, n, B, 0, n, 0.0, C, 0, n) == lib.clblasSuccess
    torch.cuda.synchronize()
    assert lib.last_gemm_variant() == name and torch.equal(C1, C2)
    assert lib.device_fault() == 0


def test_dgemm_streamk_tail_and_sgemm_splitk_are_exact(lib):
    v = _exact_gemm(lib, "d", ColumnMajor, Trans, NoTrans, 2048, 2048, 2048, seed=8020)
    assert v.endswith("+streamk_tail"), v
    v = _exact_gemm(lib, "s", ColumnMajor, NoTrans, NoTrans, 768, 768, 2048, seed=8021)
    assert "+splitk" in v, v
    v = _exact_gemm(lib, "d", ColumnMajor, NoTrans, Trans, 128, 1000, 128, seed=8022)
    assert v.startswith("dgemm_mma_tma<N,T,") and not v.startswith("dgemm_mma_tma<N,T,128>"), v     # a narrow-tile variant
    # nine 128-wide tiles with 1000 K slabs each: no whole wave at all, every SM takes an equal share of the slabs
    v = _exact_gemm(lib, "d", ColumnMajor, NoTrans, NoTrans, 300, 384, 16000, seed=8023)
    assert v == "dgemm_mma_tma<N,N,128>+streamk_tail", v


def test_triangular_16x8_kernel_through_ssyrk_and_cherk(lib):
    """Rank-k updates large enough (676 tiles, K = 1024) for the triangular instantiation of the 16 x 8 kernel."""
    n, k = 3328, 1024
    g = oracle.rng(8030, 0)
    A = g.integers(-3, 4, (n, k)).astype(np.float32)
    C = np.tril(g.integers(-3, 4, (n, n))).astype(np.float32)
    Cb = np.asfortranarray(C + np.triu(np.full((n, n), np.nan, np.float32), 1))      # the other triangle must not be touched
    dA, dC = dev(np.asfortranarray(A).ravel(order="F").copy()), dev(Cb.ravel(order="F").copy())
    st = lib.clblasSsyrk(ColumnMajor, Lower, NoTrans, n, k, 2.0, dA, 0, n, 3.0, dC, 0, n)
    torch.cuda.synchronize()
    assert st == lib.clblasSuccess and lib.last_gemm_variant() == "sgemm_nt_16x8+tri", lib.last_gemm_variant()
    got = dC.cpu().numpy().reshape(n, n).T
    want = 2.0 * (A.astype(np.float64) @ A.astype(np.float64).T) + 3.0 * C
    assert np.array_equal(np.tril(got), np.tril(want).astype(np.float32))
    assert np.all(np.isnan(got[np.triu_indices(n, 1)]))

    # CHERK: C <- alpha*A*A^H + beta*C, complex64, lower triangle; integer parts, exact
    n, k = 1792, 640
    Ar, Ai = g.integers(-3, 4, (n, k)).astype(np.float64), g.integers(-3, 4, (n, k)).astype(np.float64)
    Az = (Ar + 1j * Ai)
    Cz = np.tril(g.integers(-3, 4, (n, n)) + 1j * g.integers(-3, 4, (n, n)))
    Cz[np.diag_indices(n)] = Cz[np.diag_indices(n)].real
    store = np.asfortranarray(Cz.astype(np.complex64))
    store[np.triu_indices(n, 1)] = np.nan + 1j * np.nan
    dA = dev(np.asfortranarray(Az.astype(np.complex64)).ravel(order="F").copy().view(np.float32))
    dC = dev(store.ravel(order="F").copy().view(np.float32))
    st = lib.clblasCherk(ColumnMajor, Lower, NoTrans, n, k, 2.0, dA, 0, n, -1.0, dC, 0, n)
    torch.cuda.synchronize()
    assert st == lib.clblasSuccess and "+tri" in lib.last_gemm_variant(), lib.last_gemm_variant()
    got = dC.cpu().numpy().view(np.complex64).reshape(n, n).T
    want = 2.0 * (Az @ Az.conj().T) - Cz
    lo = np.tril_indices(n)
    assert np.array_equal(got[lo], want[lo].astype(np.complex64))
    assert lib.device_fault() == 0


@pytest.mark.parametrize("uplo", [Lower, Upper])
def test_triangular_eight_warp_stream_k_through_ssyrk_and_cherk(lib, uplo):
    """Rank-k updates with a K loop of 36 slabs or more: the eight-warp 16 x 8 stream-K kernel over the tiles that touch
    the triangle (tiles on the diagonal mask their stores).  Exact on integer inputs, the other triangle untouched."""
    n, k = 1920 + 77, 1184                     # 16 x 16 tiles with ragged edges, 136 of them in the triangle
    ld = n + 3                                 # a leading dimension that still allows 16-byte accesses (2000)
    g = oracle.rng(8060 + uplo, 0)
    A = g.integers(-3, 4, (n, k)).astype(np.float32)
    tri, other = (np.tril, np.triu_indices(n, 1)) if uplo == Lower else (np.triu, np.tril_indices(n, -1))
    C = tri(g.integers(-3, 4, (n, n))).astype(np.float32)
    Cb = np.full((ld, n), np.nan, np.float32, order="F")
    Cb[:n] = C
    Cb[:n][other] = np.nan                                                            # the other triangle must not be touched
    Ab = np.zeros((ld, k), np.float32, order="F")
    Ab[:n] = A
    dA, dC = dev(Ab.ravel(order="F").copy()), dev(Cb.ravel(order="F").copy())
    st = lib.clblasSsyrk(ColumnMajor, uplo, NoTrans, n, k, 2.0, dA, 0, ld, 3.0, dC, 0, ld)
    torch.cuda.synchronize()
    assert st == lib.clblasSuccess and lib.last_gemm_variant() == "sgemm_nt_16x8w_streamk+tri", lib.last_gemm_variant()
    got = dC.cpu().numpy().reshape(n, ld).T
    want = 2.0 * (A.astype(np.float64) @ A.astype(np.float64).T) + 3.0 * C
    assert np.array_equal(tri(got[:n]), tri(want).astype(np.float32))
    assert np.all(np.isnan(got[:n][other])) and np.all(np.isnan(got[n:]))

    # CHERK: C <- alpha*A*A^H + beta*C, complex64; integer parts, exact (the real form pairs the rows of the triangle)
    n, k = 1152, 640                           # K = 1280 in the real form
    Ar, Ai = g.integers(-3, 4, (n, k)).astype(np.float64), g.integers(-3, 4, (n, k)).astype(np.float64)
    Az = (Ar + 1j * Ai)
    Cz = tri(g.integers(-3, 4, (n, n)) + 1j * g.integers(-3, 4, (n, n)))
    Cz[np.diag_indices(n)] = Cz[np.diag_indices(n)].real
    store = np.asfortranarray(Cz.astype(np.complex64))
    other = np.triu_indices(n, 1) if uplo == Lower else np.tril_indices(n, -1)
    store[other] = np.nan + 1j * np.nan
    dA = dev(np.asfortranarray(Az.astype(np.complex64)).ravel(order="F").copy().view(np.float32))
    dC = dev(store.ravel(order="F").copy().view(np.float32))
    st = lib.clblasCherk(ColumnMajor, uplo, NoTrans, n, k, 2.0, dA, 0, n, -1.0, dC, 0, n)
    torch.cuda.synchronize()
    assert st == lib.clblasSuccess and lib.last_gemm_variant() == "sgemm_nt_16x8w_streamk+tri", lib.last_gemm_variant()
    got = dC.cpu().numpy().view(np.complex64).reshape(n, n).T
    want = 2.0 * (Az @ Az.conj().T) - Cz
    keep = np.tril_indices(n) if uplo == Lower else np.triu_indices(n)
    assert np.array_equal(got[keep], want[keep].astype(np.complex64))
    assert np.all(np.isnan(got[other].real))
    assert lib.device_fault() == 0


@pytest.mark.parametrize("uplo", [Lower, Upper])
def test_triangular_dgemm_stream_k_through_dsyrk_and_zherk(lib, uplo):
    """Double-precision rank-k updates whose tiles in the triangle would fill the last wave of CTAs only partly: all of them
    go through the FP64 stream-K kernel in equal shares.  Exact on integer inputs, the other triangle untouched."""
    n, k = 1100, 704                           # 9 x 9 tiles, 45 of them in the triangle, 44 K slabs
    g = oracle.rng(8070 + uplo, 0)
    A = g.integers(-3, 4, (n, k)).astype(np.float64)
    tri, other = (np.tril, np.triu_indices(n, 1)) if uplo == Lower else (np.triu, np.tril_indices(n, -1))
    C = tri(g.integers(-3, 4, (n, n))).astype(np.float64)
    Cb = np.asfortranarray(C.copy())
    Cb[other] = np.nan                                                               # the other triangle must not be touched
    dA, dC = dev(np.asfortranarray(A).ravel(order="F").copy()), dev(Cb.ravel(order="F").copy())
    st = lib.clblasDsyrk(ColumnMajor, uplo, NoTrans, n, k, 2.0, dA, 0, n, 3.0, dC, 0, n)
    torch.cuda.synchronize()
    assert st == lib.clblasSuccess and lib.last_gemm_variant() == "dgemm_mma_tma<N,T,128>+tri+streamk", lib.last_gemm_variant()
    got = dC.cpu().numpy().reshape(n, n).T
    want = 2.0 * (A @ A.T) + 3.0 * C
    assert np.array_equal(tri(got), tri(want))
    assert np.all(np.isnan(got[other]))
    # the same call twice gives the same bits (real-valued inputs, fixed reduction order)
    Ar = g.standard_normal((n, k))
    dA = dev(np.asfortranarray(Ar).ravel(order="F").copy())
    outs = []
    for _ in range(2):
        dC = dev(np.zeros(n * n))
        assert lib.clblasDsyrk(ColumnMajor, uplo, NoTrans, n, k, 1.0, dA, 0, n, 0.0, dC, 0, n) == lib.clblasSuccess
        outs.append(dC)
    torch.cuda.synchronize()
    assert lib.last_gemm_variant().endswith("+tri+streamk") and torch.equal(outs[0], outs[1])

    # ZHERK: complex128; the real form pairs the rows of the triangle
    n, k = 896, 512
    Az = g.integers(-3, 4, (n, k)) + 1j * g.integers(-3, 4, (n, k))
    Cz = tri(g.integers(-3, 4, (n, n)) + 1j * g.integers(-3, 4, (n, n)))
    Cz[np.diag_indices(n)] = Cz[np.diag_indices(n)].real
    store = np.asfortranarray(Cz.astype(np.complex128))
    other = np.triu_indices(n, 1) if uplo == Lower else np.tril_indices(n, -1)
    store[other] = np.nan + 1j * np.nan
    dA = dev(np.asfortranarray(Az.astype(np.complex128)).ravel(order="F").copy().view(np.float64))
    dC = dev(store.ravel(order="F").copy().view(np.float64))
    st = lib.clblasZherk(ColumnMajor, uplo, NoTrans, n, k, 2.0, dA, 0, n, -1.0, dC, 0, n)
    torch.cuda.synchronize()
    assert st == lib.clblasSuccess and lib.last_gemm_variant().endswith("+tri+streamk"), lib.last_gemm_variant()
    got = dC.cpu().numpy().view(np.complex128).reshape(n, n).T
    want = 2.0 * (Az @ Az.conj().T) - Cz
    keep = np.tril_indices(n) if uplo == Lower else np.triu_indices(n)
    assert np.array_equal(got[keep], want[keep])
    assert np.all(np.isnan(got[other].real))
    assert lib.device_fault() == 0


@pytest.mark.parametrize("nq", [2, 3, 7])
def test_gemm_over_several_queues_of_one_device(lib, nq):
    """numCommandQueues > 1: one stripe of N per queue, every queue's event recorded when its stripe is done."""
    queues = [torch.cuda.Stream() for _ in range(nq)]
    seed = 8100 + nq
    for size, (ta, tb) in zip((513, 1025), ((NoTrans, NoTrans), (Trans, ConjTrans))):
        for order in (ColumnMajor, RowMajor):
            for prec in ("s", "d"):
                seed += 1
                _exact_gemm(lib, prec, order, ta, tb, size, size, size, pad=(3, 1, 2), off=(1, 2, 3), seed=seed, queues=queues)
    assert lib.device_fault() == 0


def test_other_routines_record_every_queue_event(lib):
    """TRSM does its work on the first queue (as the reference's, src/library/blas/xtrsm.cc:1626-1629) and still
    completes the event of every queue it was given."""
    c = cases.trsm_case("d", ColumnMajor, Left, Lower, NoTrans, NonUnit, 300, 130, seed=8200)
    logical = cases.trsm_logical(c)
    A, B = cases.trsm_buffers(c, logical)
    dA, dB = dev(A), dev(B)
    queues = [torch.cuda.Stream() for _ in range(3)]
    events = [torch.cuda.Event() for _ in queues]
    for e, q in zip(events, queues):
        e.record(q)
    torch.cuda.synchronize()
    st = lib.clblasDtrsm(c["order"], c["side"], c["uplo"], c["transA"], c["diag"], c["M"], c["N"], c["alpha"], dA, c["offA"], c["lda"],
                         dB, c["offB"], c["ldb"], queues=queues, events=events)
    assert st == lib.clblasSuccess
    events[2].synchronize()                       # ordered after the solve although queue 2 did no work
    X = oracle.view(dB.cpu().numpy(), c["order"], NoTrans, c["M"], c["N"], c["ldb"], c["offB"])
    assert oracle.trsm_backward_ratio(X, c["alpha"], cases.trsm_op_triangle(c, logical[0]), logical[1], Left, np.float64) <= 1.0


def test_trsm_backward_error_against_conditioning(lib):
    """The solve multiplies by explicit inverses of the 128 x 128 diagonal blocks, so its backward error grows with
    their condition number where substitution's does not.  Unit lower triangles with off-diagonal entries of growing
    size give diagonal blocks with kappa from about 1e0 to beyond 1e10; the 4*M*u bound must hold while
    kappa <= 1e6 (measured: 3 % of the bound there) and the error may grow at most in proportion to kappa beyond."""
    n, nrhs = 512, 64
    g = oracle.rng(8300, 0)
    rows = []
    for s in (0.02, 0.05, 0.08, 0.11, 0.14, 0.18, 0.22, 0.27, 0.33, 0.4):
        L = np.tril(g.uniform(-1, 1, (n, n)), -1) * s * np.sign(g.uniform(-1, 1, (n, n))) + np.eye(n)
        L = np.tril(np.abs(L), -1) * -1.0 + np.eye(n)         # same-sign entries: the inverse grows fastest
        kappa = max(np.linalg.cond(L[b:b + 128, b:b + 128]) for b in range(0, n, 128))
        B = g.standard_normal((n, nrhs))
        dA, dB = dev(np.asfortranarray(L).ravel(order="F").copy()), dev(np.asfortranarray(B).ravel(order="F").copy())
        st = lib.clblasDtrsm(ColumnMajor, Left, Lower, NoTrans, NonUnit, n, nrhs, 1.0, dA, 0, n, dB, 0, n)
        torch.cuda.synchronize()
        assert st == lib.clblasSuccess
        X = dB.cpu().numpy().reshape(nrhs, n).T
        ratio = oracle.trsm_backward_ratio(X, 1.0, L, B, Left, np.float64)
        rows.append((kappa, ratio))
    print("kappa of the worst diagonal block -> backward error / (4*M*u):", [(f"{k:.1e}", f"{r:.3g}") for k, r in rows])
    for kappa, ratio in rows:
        if kappa <= 1e6:
            assert ratio <= 1.0, (kappa, ratio)
        assert ratio <= max(1.0, kappa * 1e-6), (kappa, ratio)
