// Symmetric rank-k update: C <- alpha * op(A) * op(A)^T + beta * C on one triangle of the N x N matrix C.
//
// Replaces clblasSsyrk / clblasDsyrk (src/clBLAS.h:8279-8296, :8351-8368; src/library/blas/xsyrk.c), which
// the reference serves with its run-time generated legacy kernels.  Here the update is ONE launch of
// the library's GEMM kernels in their triangular mode (GemmProblem::tri): both operands are the same
// stored matrix, tiles entirely outside the referenced triangle exit at once, tiles on the diagonal
// mask their stores, so the other triangle of C is never read or written and only about half of the
// N*N*K products are formed.
#include "common.h"

#include <algorithm>

namespace cb200 {

namespace {

// C[i,j] = beta*C[i,j] for (i,j) in the referenced triangle of the n x n matrix; beta == 0 never reads C.
template <typename T>
__global__ void __launch_bounds__(256) tri_scale_kernel(T* __restrict__ C, size_t ldc, size_t n, bool lower, T beta)
{
    const size_t total = n * n;
    for (size_t e = (size_t)blockIdx.x * 256 + threadIdx.x; e < total; e += (size_t)gridDim.x * 256) {
        const size_t i = e % n, j = e / n;
        if (lower ? i < j : i > j) continue;
        T* c = C + i + j * ldc;
        *c = beta != T(0) ? beta * *c : T(0);
    }
}

}  // namespace

namespace {

template <typename T>
cudaError_t tri_scale(bool lower, size_t N, T beta, T* C, size_t ldc, cudaStream_t s)
{
    if (beta == T(1)) return cudaSuccess;
    const unsigned blocks = (unsigned)std::min<size_t>((N * N + 255) / 256, (size_t)sm_count() * 8);
    tri_scale_kernel<T><<<blocks, 256, 0, s>>>(C, ldc, N, lower, beta);
    count_launch();
    return cudaGetLastError();
}

// op(X) = X (N x K): X * Y^T is (no-trans, trans); op(X) = X^T with X stored K x N: (trans, no-trans)
template <typename T>
cudaError_t tri_product(bool lower, bool trans, size_t N, size_t K, T alpha, const T* X, size_t ldx, const T* Y, size_t ldy,
                        T beta, T* C, size_t ldc, cudaStream_t s)
{
    GemmProblem<T> p;
    p.ta = trans; p.tb = !trans; p.M = N; p.N = N; p.K = K; p.alpha = alpha; p.A = X; p.lda = ldx;
    p.B = Y; p.ldb = ldy; p.beta = beta; p.C = C; p.ldc = ldc;
    p.tri = lower ? TRI_LOWER : TRI_UPPER;
    return gemm_colmajor<T>(p, s);
}

}  // namespace

template <typename T>
cudaError_t syrk_colmajor(bool lower, bool trans, size_t N, size_t K, T alpha, const T* A, size_t lda, T beta,
                          T* C, size_t ldc, cudaStream_t s)
{
    if (N == 0) return cudaSuccess;
    // BLAS semantics: K == 0 or alpha == 0 scales the triangle of C by beta, A is not referenced
    if (K == 0 || alpha == T(0)) return tri_scale<T>(lower, N, beta, C, ldc, s);
    return tri_product<T>(lower, trans, N, K, alpha, A, lda, A, lda, beta, C, ldc, s);
}

// Symmetric rank-2k update (clblasSsyr2k / clblasDsyr2k, src/clBLAS.h:8568-8589, :8648-8669;
// src/library/blas/xsyr2k.c): C <- alpha*op(A)*op(B)^T + alpha*op(B)*op(A)^T + beta*C on one triangle,
// as two triangular products, the second accumulating onto the first.
template <typename T>
cudaError_t syr2k_colmajor(bool lower, bool trans, size_t N, size_t K, T alpha, const T* A, size_t lda, const T* B,
                           size_t ldb, T beta, T* C, size_t ldc, cudaStream_t s)
{
    if (N == 0) return cudaSuccess;
    if (K == 0 || alpha == T(0)) return tri_scale<T>(lower, N, beta, C, ldc, s);
    cudaError_t e = tri_product<T>(lower, trans, N, K, alpha, A, lda, B, ldb, beta, C, ldc, s);
    if (e != cudaSuccess) return e;
    return tri_product<T>(lower, trans, N, K, alpha, B, ldb, A, lda, T(1), C, ldc, s);
}

template cudaError_t syrk_colmajor<float>(bool, bool, size_t, size_t, float, const float*, size_t, float, float*, size_t, cudaStream_t);
template cudaError_t syrk_colmajor<double>(bool, bool, size_t, size_t, double, const double*, size_t, double, double*, size_t, cudaStream_t);
template cudaError_t syr2k_colmajor<float>(bool, bool, size_t, size_t, float, const float*, size_t, const float*, size_t, float, float*, size_t, cudaStream_t);
template cudaError_t syr2k_colmajor<double>(bool, bool, size_t, size_t, double, const double*, size_t, const double*, size_t, double, double*, size_t, cudaStream_t);

}  // namespace cb200
