// Complex symmetric / Hermitian level-3 routines on the complex GEMM of cgemm.cu:
//   clblasCsyrk / Zsyrk (src/clBLAS.h:8417, :8485), clblasCherk / Zherk (:9389, :9458),
//   clblasCsyr2k / Zsyr2k (:8722, :8798), clblasCher2k / Zher2k (:9545, :9623),
//   clblasCsymm / Zsymm (:9052, :9124), clblasChemm / Zhemm (:9224, :9305).
// Rank-k updates are one (rank-2k: two) complex GEMM launch in the triangular mode, where both real rows of a
// complex row share its place in the triangle (TRI_PAIRED_ROWS); the other triangle of C is never touched.
// Hermitian variants conjugate through the GEMM's ConjTrans operand and end by clearing the imaginary parts of
// the diagonal.  SYMM / HEMM expand the stored triangle of A into a dense matrix once and call the GEMM.
#include "common.h"

#include <algorithm>

namespace cb200 {

namespace {

template <typename R> struct Cx;
template <> struct Cx<float> { using type = float2; };
template <> struct Cx<double> { using type = double2; };

inline unsigned grid_for(size_t total) { return (unsigned)std::min<size_t>((total + 255) / 256, (size_t)sm_count() * 16); }

// C[i,j] <- beta*C[i,j] on the triangle (beta == 0: zeros, C not read); diagonal imaginary parts cleared on request.
template <typename R>
__global__ void __launch_bounds__(256) ctri_scale_kernel(R* __restrict__ C, size_t ldc, size_t n, bool lower, R br, R bi,
                                                         bool scale, bool zero_diag_imag)
{
    using R2 = typename Cx<R>::type;
    const size_t total = n * n;
    const bool zero = (br == R(0) && bi == R(0));
    for (size_t e = (size_t)blockIdx.x * 256 + threadIdx.x; e < total; e += (size_t)gridDim.x * 256) {
        const size_t i = e % n, j = e / n;
        if (lower ? i < j : i > j) continue;
        if (!scale && i != j) continue;
        R2* c = reinterpret_cast<R2*>(C + 2 * (i + j * ldc));
        R2 v;
        if (scale && zero) { v.x = R(0); v.y = R(0); }
        else {
            v = *c;
            if (scale) { const R x = br * v.x - bi * v.y, y = br * v.y + bi * v.x; v.x = x; v.y = y; }
        }
        if (zero_diag_imag && i == j) v.y = R(0);
        *c = v;
    }
}

// Dense n x n matrix from the stored triangle of a symmetric (mirror = same value) or Hermitian (mirror = conjugate,
// real diagonal) matrix; 32 x 32 tiles through shared memory, as symm.cu does for real matrices.
template <typename R, bool HERM>
__global__ void __launch_bounds__(256) csymmetrize_kernel(const R* __restrict__ A, size_t lda, R* __restrict__ F, size_t ldf,
                                                          size_t n, bool lower)
{
    using R2 = typename Cx<R>::type;
    __shared__ R2 tile[32][33];
    const size_t bi = blockIdx.x, bj = blockIdx.y;
    const int tx = threadIdx.x % 32, ty = threadIdx.x / 32;
    const bool stored = lower ? bi >= bj : bi <= bj;
    const size_t si = stored ? bi : bj, sj = stored ? bj : bi;
    for (int r = ty; r < 32; r += 8) {
        const size_t i = si * 32 + tx, j = sj * 32 + r;
        const bool in_tri = lower ? i >= j : i <= j;
        R2 v; v.x = R(0); v.y = R(0);
        if (i < n && j < n && in_tri) v = *reinterpret_cast<const R2*>(A + 2 * (i + j * lda));
        tile[r][tx] = v;
    }
    __syncthreads();
    for (int r = ty; r < 32; r += 8) {
        const size_t i = bi * 32 + tx, j = bj * 32 + r;
        if (i >= n || j >= n) continue;
        bool direct;                                   // entry taken as stored, or mirrored
        if (bi == bj) direct = lower ? tx >= r : tx <= r; else direct = stored;
        R2 v = direct ? tile[r][tx] : tile[tx][r];
        if (HERM) {
            if (!direct) v.y = -v.y;
            if (i == j) v.y = R(0);
        }
        *reinterpret_cast<R2*>(F + 2 * (i + j * ldf)) = v;
    }
}

}  // namespace

template <typename R>
cudaError_t complex_tri_scale(bool lower, size_t N, R br, R bi, R* C, size_t ldc, bool zero_diag_imag, cudaStream_t s)
{
    const bool scale = !(br == R(1) && bi == R(0));
    if (N == 0 || (!scale && !zero_diag_imag)) return cudaSuccess;
    ctri_scale_kernel<R><<<grid_for(N * N), 256, 0, s>>>(C, ldc, N, lower, br, bi, scale, zero_diag_imag);
    count_launch();
    return cudaGetLastError();
}

template <typename R>
cudaError_t csyrk_colmajor(bool herm, bool lower, int op, size_t N, size_t K, R ar, R ai, const R* A, size_t lda,
                           R br, R bi, R* C, size_t ldc, cudaStream_t s)
{
    if (N == 0) return cudaSuccess;
    const int tri = lower ? TRI_LOWER : TRI_UPPER;
    if (K == 0 || (ar == R(0) && ai == R(0))) return complex_tri_scale<R>(lower, N, br, bi, C, ldc, herm, s);
    // op(A) op(A)^T (SYRK) or op(A) op(A)^H (HERK): the second operand is the same matrix, transposed the other way
    const int other = herm ? 2 : 1;
    cudaError_t e = op == 0 ? cgemm_colmajor<R>(0, other, N, N, K, ar, ai, A, lda, A, lda, br, bi, C, ldc, s, tri)
                            : cgemm_colmajor<R>(other, 0, N, N, K, ar, ai, A, lda, A, lda, br, bi, C, ldc, s, tri);
    if (e != cudaSuccess || !herm) return e;
    return complex_tri_scale<R>(lower, N, R(1), R(0), C, ldc, true, s);
}

template <typename R>
cudaError_t csyr2k_colmajor(bool herm, bool lower, int op, size_t N, size_t K, R ar, R ai, const R* A, size_t lda,
                            const R* B, size_t ldb, R br, R bi, R* C, size_t ldc, cudaStream_t s)
{
    if (N == 0) return cudaSuccess;
    const int tri = lower ? TRI_LOWER : TRI_UPPER;
    if (K == 0 || (ar == R(0) && ai == R(0))) return complex_tri_scale<R>(lower, N, br, bi, C, ldc, herm, s);
    const int other = herm ? 2 : 1;
    const R ai2 = herm ? -ai : ai;                  // HER2K: the second product carries conj(alpha)
    cudaError_t e;
    if (op == 0) {
        e = cgemm_colmajor<R>(0, other, N, N, K, ar, ai, A, lda, B, ldb, br, bi, C, ldc, s, tri);
        if (e == cudaSuccess) e = cgemm_colmajor<R>(0, other, N, N, K, ar, ai2, B, ldb, A, lda, R(1), R(0), C, ldc, s, tri);
    } else {
        e = cgemm_colmajor<R>(other, 0, N, N, K, ar, ai, A, lda, B, ldb, br, bi, C, ldc, s, tri);
        if (e == cudaSuccess) e = cgemm_colmajor<R>(other, 0, N, N, K, ar, ai2, B, ldb, A, lda, R(1), R(0), C, ldc, s, tri);
    }
    if (e != cudaSuccess || !herm) return e;
    return complex_tri_scale<R>(lower, N, R(1), R(0), C, ldc, true, s);
}

template <typename R>
cudaError_t csymm_colmajor(bool herm, bool right, bool lower, size_t M, size_t N, R ar, R ai, const R* A, size_t lda,
                           const R* B, size_t ldb, R br, R bi, R* C, size_t ldc, cudaStream_t s)
{
    if (M == 0 || N == 0) return cudaSuccess;
    if (ar == R(0) && ai == R(0)) return complex_scale<R>(C, ldc, M, N, br, bi, s);
    const size_t n = right ? N : M;
    constexpr size_t Q = 8 / sizeof(R);             // complex elements per 16 bytes
    const size_t ldf = (n + Q - 1) / Q * Q;
    const size_t tiles = (n + 31) / 32;
    if (tiles > 65535) return cudaErrorNotSupported;
    R* F = nullptr;
    cudaError_t e = ws_alloc(reinterpret_cast<void**>(&F), 2 * ldf * n * sizeof(R), s);
    if (e != cudaSuccess) return e;
    if (herm) csymmetrize_kernel<R, true><<<dim3((unsigned)tiles, (unsigned)tiles), 256, 0, s>>>(A, lda, F, ldf, n, lower);
    else      csymmetrize_kernel<R, false><<<dim3((unsigned)tiles, (unsigned)tiles), 256, 0, s>>>(A, lda, F, ldf, n, lower);
    count_launch();
    e = cudaGetLastError();
    if (e == cudaSuccess) {
        if (right) e = cgemm_colmajor<R>(0, 0, M, N, n, ar, ai, B, ldb, F, ldf, br, bi, C, ldc, s);
        else       e = cgemm_colmajor<R>(0, 0, M, N, n, ar, ai, F, ldf, B, ldb, br, bi, C, ldc, s);
    }
    const cudaError_t e2 = ws_free(F, s);
    return e != cudaSuccess ? e : e2;
}

#define INST(R)                                                                                                          \
    template cudaError_t complex_tri_scale<R>(bool, size_t, R, R, R*, size_t, bool, cudaStream_t);                       \
    template cudaError_t csyrk_colmajor<R>(bool, bool, int, size_t, size_t, R, R, const R*, size_t, R, R, R*, size_t,     \
                                           cudaStream_t);                                                                \
    template cudaError_t csyr2k_colmajor<R>(bool, bool, int, size_t, size_t, R, R, const R*, size_t, const R*, size_t, R, \
                                            R, R*, size_t, cudaStream_t);                                                \
    template cudaError_t csymm_colmajor<R>(bool, bool, bool, size_t, size_t, R, R, const R*, size_t, const R*, size_t, R, \
                                           R, R*, size_t, cudaStream_t);
INST(float)
INST(double)
#undef INST

}  // namespace cb200
