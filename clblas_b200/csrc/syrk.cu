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

template <typename T>
cudaError_t syrk_colmajor(bool lower, bool trans, size_t N, size_t K, T alpha, const T* A, size_t lda, T beta,
                          T* C, size_t ldc, cudaStream_t s)
{
    if (N == 0) return cudaSuccess;
    if (K == 0 || alpha == T(0)) {
        // BLAS semantics: the triangle of C is scaled by beta, A is not referenced
        if (beta == T(1)) return cudaSuccess;
        const unsigned blocks = (unsigned)std::min<size_t>((N * N + 255) / 256, (size_t)sm_count() * 8);
        tri_scale_kernel<T><<<blocks, 256, 0, s>>>(C, ldc, N, lower, beta);
        count_launch();
        return cudaGetLastError();
    }
    // op(A) = A (N x K, rows contiguous in N): A * A^T is (no-trans, trans); op(A) = A^T with A stored K x N: (trans, no-trans)
    GemmProblem<T> p;
    p.ta = trans; p.tb = !trans; p.M = N; p.N = N; p.K = K; p.alpha = alpha; p.A = A; p.lda = lda;
    p.B = A; p.ldb = lda; p.beta = beta; p.C = C; p.ldc = ldc;
    p.tri = lower ? TRI_LOWER : TRI_UPPER;
    return gemm_colmajor<T>(p, s);
}

template cudaError_t syrk_colmajor<float>(bool, bool, size_t, size_t, float, const float*, size_t, float, float*, size_t, cudaStream_t);
template cudaError_t syrk_colmajor<double>(bool, bool, size_t, size_t, double, const double*, size_t, double, double*, size_t, cudaStream_t);

}  // namespace cb200
