"""The benchmark's workloads at their full sizes on one GPU (DGEMM T/N 8192^3, DTRSM 8192 x 16384, SGEMM N/T 32768^3).

A full float64 host product is out of reach at these sizes, so each run is checked through
(a) sampled rows x columns of the result against a float64 host evaluation of the SAME device data,
with the stated bound (GEMM 4*K*u on |alpha||A||B| + |beta||C|; TRSM backward error 4*M*u), and
(b) size-independent properties evaluated on the device: exact scaling by powers of two, a checksum of
checksums, NaN canaries (beta = 0 must not read C; the garbage triangle of A must not be read)."""
import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu

U32, U64 = 2.0 ** -24, 2.0 ** -53


def _gen(n, dtype, seed, kind):
    g = torch.Generator(device="cuda")
    g.manual_seed(seed)
    t = torch.empty(n, dtype=dtype, device="cuda")
    return t.normal_(generator=g) if kind == "normal" else t.uniform_(-1.0, 1.0, generator=g)


def _sample(n, count, seed, always=()):
    r = np.random.Generator(np.random.Philox(key=[seed, 0])).choice(n, size=count, replace=False)
    return np.unique(np.concatenate([r, np.array(always, dtype=r.dtype)]))


def _ratio(got, exact, denom, K, u):
    denom = np.where(denom == 0, np.finfo(np.float64).tiny, denom)
    return float(np.max(np.abs(got.astype(np.float64) - exact) / denom) / (4.0 * K * u))


def test_config2_dgemm_tn_8192(lib):
    """DGEMM column-major T/N, M=N=K=8192, normal(0,1), alpha=beta=1, tight leading dimensions."""
    n = 8192
    A, B, C0 = (_gen(n * n, torch.float64, s, "normal") for s in (1, 2, 3))
    C = C0.clone()
    st = lib.clblasDgemm(lib.clblasColumnMajor, lib.clblasTrans, lib.clblasNoTrans, n, n, n, 1.0, A, 0, n, B, 0, n, 1.0, C, 0, n)
    assert st == lib.clblasSuccess and lib.last_gemm_kernel() == "dgemm_mma_tma"
    rows, cols = _sample(n, 48, 10, always=(0, n - 1)), _sample(n, 48, 11, always=(0, n - 1))
    ri, ci = torch.from_numpy(rows).cuda(), torch.from_numpy(cols).cuda()
    Av = A.view(n, n)[ri].cpu().numpy()                    # stored A is K x M column-major: row i of op(A) = column i
    Bv = B.view(n, n)[ci].cpu().numpy()                    # column j of B
    C0s = C0.view(n, n)[ci][:, ri].cpu().numpy().T         # C(i, j) = flat[i + j*n]
    Cs = C.view(n, n)[ci][:, ri].cpu().numpy().T
    exact = Av @ Bv.T + C0s
    denom = np.abs(Av) @ np.abs(Bv).T + np.abs(C0s)
    assert _ratio(Cs, exact, denom, n, U64) <= 1.0
    # property: scaling alpha by 2 (beta = 0) doubles every entry exactly
    C1, C2 = torch.empty_like(C), torch.empty_like(C)
    lib.clblasDgemm(lib.clblasColumnMajor, lib.clblasTrans, lib.clblasNoTrans, n, n, n, 1.0, A, 0, n, B, 0, n, 0.0, C1, 0, n)
    lib.clblasDgemm(lib.clblasColumnMajor, lib.clblasTrans, lib.clblasNoTrans, n, n, n, 2.0, A, 0, n, B, 0, n, 0.0, C2, 0, n)
    assert torch.equal(C2, 2.0 * C1)
    # property: checksum of checksums, sum_ij C1 = sum_k (sum_i A[k,i]) (sum_j B[k,j])
    lhs = C1.sum().item()
    rhs = (A.view(n, n).sum(dim=0) * B.view(n, n).sum(dim=0)).sum().item()
    scale = (A.view(n, n).abs().sum(dim=0) * B.view(n, n).abs().sum(dim=0)).sum().item()
    assert abs(lhs - rhs) <= 1e-9 * scale
    assert lib.device_fault() == 0


def test_config4_dtrsm_left_lower_8192x16384(lib):
    """DTRSM column-major Left/Lower/NoTrans/NonUnit: A 8192^2 (diag U[1,2], strict lower U[-1,1]/8192,
    strict upper = NaN and huge values that must never be read), B 8192 x 16384 normal(0,1), alpha=1."""
    M, N = 8192, 16384
    A = _gen(M * M, torch.float64, 4, "uniform") / M
    Av = A.view(M, M)                                      # Av[j, i] = A(i, j)
    Av.diagonal().copy_(_gen(M, torch.float64, 5, "uniform") * 0.5 + 1.5)
    iu = torch.triu_indices(M, M, offset=1, device="cuda")
    Av[iu[1], iu[0]] = float("nan")
    Av[iu[1][::7], iu[0][::7]] = 1e300
    del iu
    B0 = _gen(M * N, torch.float64, 6, "normal")
    X = B0.clone()
    st = lib.clblasDtrsm(lib.clblasColumnMajor, lib.clblasLeft, lib.clblasLower, lib.clblasNoTrans, lib.clblasNonUnit,
                         M, N, 1.0, A, 0, M, X, 0, M)
    assert st == lib.clblasSuccess
    assert bool(torch.isfinite(X).all())
    cols = _sample(N, 24, 12, always=(0, N - 1, 2047, 2048))
    ci = torch.from_numpy(cols).cuda()
    Xs = X.view(N, M)[ci].cpu().numpy().T                   # M x len(cols)
    Bs = B0.view(N, M)[ci].cpu().numpy().T
    T = np.tril(np.nan_to_num(Av.cpu().numpy().T, nan=0.0))
    assert oracle.trsm_backward_ratio(Xs, 1.0, T, Bs, oracle.Left, np.float64) <= 1.0
    # property: right-hand-side columns are independent -- solving a slab alone gives the same solution.  Not bit
    # for bit: the GEMM kernels walk K forwards or backwards depending on a tile's place in the grid, and the
    # grid depends on N, so only the rounding differs.
    Y = B0[: M * 256].clone()
    lib.clblasDtrsm(lib.clblasColumnMajor, lib.clblasLeft, lib.clblasLower, lib.clblasNoTrans, lib.clblasNonUnit,
                    M, 256, 1.0, A, 0, M, Y, 0, M)
    ref = X[: M * 256]
    assert float((Y - ref).abs().max()) <= 16 * M * 2.0 ** -53 * float(ref.abs().max())
    # and the same call twice is bit-identical
    Y2 = B0[: M * 256].clone()
    lib.clblasDtrsm(lib.clblasColumnMajor, lib.clblasLeft, lib.clblasLower, lib.clblasNoTrans, lib.clblasNonUnit,
                    M, 256, 1.0, A, 0, M, Y2, 0, M)
    assert torch.equal(Y, Y2)
    assert lib.device_fault() == 0


def test_config5_sgemm_nt_32768(lib):
    """SGEMM column-major N/T, M=N=K=32768, U[-1,1], alpha=1, beta=0, C pre-filled with NaN."""
    n = 32768
    free, _ = torch.cuda.mem_get_info()
    if free < 3 * 4 * n * n + (2 << 30):
        pytest.skip("not enough free device memory for three 4 GiB matrices")
    A, B = _gen(n * n, torch.float32, 7, "uniform"), _gen(n * n, torch.float32, 8, "uniform")
    C = torch.full((n * n,), float("nan"), dtype=torch.float32, device="cuda")
    st = lib.clblasSgemm(lib.clblasColumnMajor, lib.clblasNoTrans, lib.clblasTrans, n, n, n, 1.0, A, 0, n, B, 0, n, 0.0, C, 0, n)
    assert st == lib.clblasSuccess and lib.last_gemm_kernel() == "sgemm_ffma_tma"
    assert not bool(torch.isnan(C).any())                  # beta = 0 never reads C
    seams = [4096 * k + d for k in range(1, 8) for d in (-1, 0)]       # shard seams of the 2/4/8-GPU split
    rows, cols = _sample(n, 40, 13, always=(0, n - 1)), _sample(n, 40, 14, always=[0, n - 1] + seams)
    ri, ci = torch.from_numpy(rows).cuda(), torch.from_numpy(cols).cuda()
    Ar = A.view(n, n)[:, ri].cpu().numpy().astype(np.float64).T      # A(i, k) = flat[i + k*n] -> rows x K
    Bc = B.view(n, n)[:, ci].cpu().numpy().astype(np.float64).T      # B(j, k) = flat[j + k*n] -> cols x K
    Cs = C.view(n, n)[ci][:, ri].cpu().numpy().T
    exact, denom = Ar @ Bc.T, np.abs(Ar) @ np.abs(Bc).T
    assert _ratio(Cs, exact, denom, n, U32) <= 1.0
    # property: checksum of checksums in float64 on the device
    lhs = C.sum(dtype=torch.float64).item()
    ca, cb_ = A.view(n, n).sum(dim=1, dtype=torch.float64), B.view(n, n).sum(dim=1, dtype=torch.float64)
    rhs = (ca * cb_).sum().item()
    scale = (A.view(n, n).abs().sum(dim=1, dtype=torch.float64) * B.view(n, n).abs().sum(dim=1, dtype=torch.float64)).sum().item()
    assert abs(lhs - rhs) <= 4 * n * U32 * scale
    assert lib.device_fault() == 0
