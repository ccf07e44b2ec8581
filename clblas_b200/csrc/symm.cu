// Symmetric matrix multiply: C <- alpha*A*B + beta*C (Left, A is M x M) or C <- alpha*B*A + beta*C
// (Right, A is N x N), where only the `uplo` triangle of the symmetric matrix A is stored.
//
// Replaces clblasSsymm / clblasDsymm (src/clBLAS.h:8898-8919, :8979-9000; src/library/blas/xsymm.c, which
// also turns SYMM into GEMM calls: SYMM_USING_GEMM).  Here the stored triangle is expanded once into a
// dense symmetric matrix in a stream-ordered workspace (n*n elements, one coalesced pass that reads
// only the referenced triangle), then ONE GEMM on the library's kernels forms the product: the
// expansion moves 2*n*n elements against 2*n*n*other flops of the product.
#include "common.h"

namespace cb200 {

namespace {

// 32 x 32 tiles; tile (bi, bj) of the dense output comes from the stored tile (bi, bj) when that lies
// in the referenced triangle, else from the mirror tile (bj, bi) read through shared memory.  Tiles on
// the diagonal take each entry from whichever of (i, j) / (j, i) is stored.
template <typename T>
__global__ void __launch_bounds__(256) symmetrize_kernel(const T* __restrict__ A, size_t lda, T* __restrict__ F, size_t ldf,
                                                         size_t n, bool lower)
{
    __shared__ T tile[32][33];
    const size_t bi = blockIdx.x, bj = blockIdx.y;
    const int tx = threadIdx.x % 32, ty = threadIdx.x / 32;      // 32 x 8
    const bool stored = lower ? bi >= bj : bi <= bj;             // tile (bi, bj) holds referenced entries
    const size_t si = stored ? bi : bj, sj = stored ? bj : bi;   // source tile
    for (int r = ty; r < 32; r += 8) {
        const size_t i = si * 32 + tx, j = sj * 32 + r;
        const bool in_tri = lower ? i >= j : i <= j;
        tile[r][tx] = (i < n && j < n && in_tri) ? A[i + j * lda] : T(0);   // tile[col][row] of the source tile
    }
    __syncthreads();
    for (int r = ty; r < 32; r += 8) {
        const size_t i = bi * 32 + tx, j = bj * 32 + r;
        if (i >= n || j >= n) continue;
        T v;
        if (bi == bj) {
            const bool in_tri = lower ? tx >= r : tx <= r;
            v = in_tri ? tile[r][tx] : tile[tx][r];
        } else {
            v = stored ? tile[r][tx] : tile[tx][r];
        }
        F[i + j * ldf] = v;
    }
}

}  // namespace

template <typename T>
cudaError_t symm_colmajor(bool right, bool lower, size_t M, size_t N, T alpha, const T* A, size_t lda, const T* B, size_t ldb,
                          T beta, T* C, size_t ldc, cudaStream_t s)
{
    if (M == 0 || N == 0) return cudaSuccess;
    GemmProblem<T> p;
    p.ta = false; p.tb = false; p.M = M; p.N = N; p.alpha = alpha; p.beta = beta; p.C = C; p.ldc = ldc;
    if (alpha == T(0)) {
        // C <- beta*C; neither A nor B is referenced
        p.K = 0; p.A = A; p.lda = lda; p.B = B; p.ldb = ldb;
        return gemm_colmajor<T>(p, s);
    }
    const size_t n = right ? N : M;
    constexpr size_t Q = 16 / sizeof(T);
    const size_t ldf = (n + Q - 1) / Q * Q;
    if (n > 0xFFFFu * 32u) return cudaErrorNotSupported;
    T* F = nullptr;
    cudaError_t e = ws_alloc(reinterpret_cast<void**>(&F), ldf * n * sizeof(T), s);
    if (e != cudaSuccess) return e;
    const unsigned tiles = (unsigned)((n + 31) / 32);
    symmetrize_kernel<T><<<dim3(tiles, tiles), 256, 0, s>>>(A, lda, F, ldf, n, lower);
    count_launch();
    e = cudaGetLastError();
    if (e == cudaSuccess) {
        p.K = n;
        if (right) { p.A = B; p.lda = ldb; p.B = F; p.ldb = ldf; }
        else       { p.A = F; p.lda = ldf; p.B = B; p.ldb = ldb; }
        e = gemm_colmajor<T>(p, s);
    }
    const cudaError_t e2 = ws_free(F, s);
    return e != cudaSuccess ? e : e2;
}

template cudaError_t symm_colmajor<float>(bool, bool, size_t, size_t, float, const float*, size_t, const float*, size_t, float, float*, size_t, cudaStream_t);
template cudaError_t symm_colmajor<double>(bool, bool, size_t, size_t, double, const double*, size_t, const double*, size_t, double, double*, size_t, cudaStream_t);

}  // namespace cb200
