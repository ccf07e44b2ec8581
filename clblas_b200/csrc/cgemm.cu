// Complex GEMM (clblasCgemm / clblasZgemm, src/clBLAS.h:7538-7560, :7614-7636; src/library/blas/xgemm.cc:788-905)
// on the real GEMM kernels.
//
// A column-major complex matrix with interleaved (re, im) storage IS a real matrix with twice the rows
// and twice the leading dimension.  With every complex entry a of alpha*op(A) written as the 2 x 2
// real block [[re, -im], [im, re]], the complex product is one REAL product
//
//     C_real (2M x N)  =  A~ (2M x 2K)  *  B_real (2K x N)  +  beta * C_real
//
// of exactly the complex flop count (8*M*N*K), which runs on the FP64 tensor-core / packed-FP32 kernels
// at their real-GEMM rate.  B and C are used where they lie (no copy) when B is not transposed; a
// transposed or conjugated B is split once into a planar N x 2K real matrix (coalesced, no
// transposition); A~ is written once (twice the size of A) in whichever orientation needs no
// transposition.  beta with a non-zero imaginary part is applied to C by a scaling pass first.
#include "common.h"

#include <algorithm>

namespace cb200 {

namespace {

template <typename R> struct Pair;
template <> struct Pair<float> { using type = float2; };
template <> struct Pair<double> { using type = double2; };

template <typename R>
__device__ __forceinline__ typename Pair<R>::type mk2(R x, R y)
{
    typename Pair<R>::type v;
    v.x = x; v.y = y;
    return v;
}

// A~ from alpha*op(A).  TRANS == 0: A stored M x K (rows contiguous), A~ stored 2M x 2K.
// TRANS != 0: A stored K x M, op(A) = A^T (or A^H when conj); A~^T stored 2K x 2M.
// In both cases f runs along the contiguous direction of the stored matrix (extent nf), g along the other.
template <typename R, bool TRANS>
__global__ void __launch_bounds__(256) expand_a_kernel(const R* __restrict__ A, size_t lda, R* __restrict__ E, size_t lde,
                                                       size_t nf, size_t ng, R ar, R ai, bool conj)
{
    using R2 = typename Pair<R>::type;
    const size_t total = nf * ng;
    for (size_t e = (size_t)blockIdx.x * 256 + threadIdx.x; e < total; e += (size_t)gridDim.x * 256) {
        const size_t f = e % nf, g = e / nf;
        const R2 a = *reinterpret_cast<const R2*>(A + 2 * (f + g * lda));
        const R xi = conj ? -a.y : a.y;
        const R vr = ar * a.x - ai * xi, vi = ar * xi + ai * a.x;
        R* c0 = E + 2 * f + (2 * g) * lde;
        R* c1 = c0 + lde;
        if (!TRANS) {
            // rows 2i, 2i+1 of columns 2k and 2k+1: (re, im) and (-im, re)
            *reinterpret_cast<R2*>(c0) = mk2<R>(vr, vi);
            *reinterpret_cast<R2*>(c1) = mk2<R>(-vi, vr);
        } else {
            // rows 2k, 2k+1 of columns 2i and 2i+1 of the transposed block matrix: (re, -im) and (im, re)
            *reinterpret_cast<R2*>(c0) = mk2<R>(vr, -vi);
            *reinterpret_cast<R2*>(c1) = mk2<R>(vi, vr);
        }
    }
}

// Stored B is N x K complex (op(B) = B^T or B^H).  P (N x 2K real): column 2k = Re, column 2k+1 = +-Im.
template <typename R>
__global__ void __launch_bounds__(256) planar_b_kernel(const R* __restrict__ B, size_t ldb, R* __restrict__ P, size_t ldp,
                                                       size_t N, size_t K, bool conj)
{
    using R2 = typename Pair<R>::type;
    const size_t total = N * K;
    for (size_t e = (size_t)blockIdx.x * 256 + threadIdx.x; e < total; e += (size_t)gridDim.x * 256) {
        const size_t j = e % N, k = e / N;
        const R2 b = *reinterpret_cast<const R2*>(B + 2 * (j + k * ldb));
        P[j + (2 * k) * ldp] = b.x;
        P[j + (2 * k + 1) * ldp] = conj ? -b.y : b.y;
    }
}

// C <- beta*C for complex beta; beta == 0 stores zeros without reading C.
template <typename R>
__global__ void __launch_bounds__(256) cscale_kernel(R* __restrict__ C, size_t ldc, size_t M, size_t N, R br, R bi)
{
    using R2 = typename Pair<R>::type;
    const size_t total = M * N;
    const bool zero = (br == R(0) && bi == R(0));
    for (size_t e = (size_t)blockIdx.x * 256 + threadIdx.x; e < total; e += (size_t)gridDim.x * 256) {
        R2* c = reinterpret_cast<R2*>(C + 2 * (e % M + (e / M) * ldc));
        if (zero) { *c = mk2<R>(R(0), R(0)); continue; }
        const R2 v = *c;
        *c = mk2<R>(br * v.x - bi * v.y, br * v.y + bi * v.x);
    }
}

inline unsigned grid_for(size_t total) { return (unsigned)std::min<size_t>((total + 255) / 256, (size_t)sm_count() * 16); }

// dst (cols x rows complex, column-major) = src^T (src rows x cols complex), through 32 x 32 shared tiles
template <typename R>
__global__ void __launch_bounds__(256) ctranspose_kernel(const R* __restrict__ src, size_t lds, R* __restrict__ dst, size_t ldd,
                                                         size_t rows, size_t cols)
{
    using R2 = typename Pair<R>::type;
    __shared__ R2 tile[32][33];
    const size_t r0 = (size_t)blockIdx.x * 32, c0 = (size_t)blockIdx.y * 32;
    const int tx = threadIdx.x % 32, ty = threadIdx.x / 32;
    for (int c = ty; c < 32; c += 8)
        if (r0 + tx < rows && c0 + c < cols) tile[c][tx] = *reinterpret_cast<const R2*>(src + 2 * (r0 + tx + (c0 + c) * lds));
    __syncthreads();
    for (int r = ty; r < 32; r += 8)
        if (c0 + tx < cols && r0 + r < rows) *reinterpret_cast<R2*>(dst + 2 * (c0 + tx + (r0 + r) * ldd)) = tile[tx][r];
}

}  // namespace

template <typename R>
cudaError_t complex_scale(R* C, size_t ldc, size_t M, size_t N, R br, R bi, cudaStream_t s)
{
    if (M == 0 || N == 0 || (br == R(1) && bi == R(0))) return cudaSuccess;
    cscale_kernel<R><<<grid_for(M * N), 256, 0, s>>>(C, ldc, M, N, br, bi);
    count_launch();
    return cudaGetLastError();
}

template <typename R>
cudaError_t complex_transpose(R* dst, size_t ldd, const R* src, size_t lds, size_t rows, size_t cols, cudaStream_t s)
{
    if (rows == 0 || cols == 0) return cudaSuccess;
    const size_t bx = (rows + 31) / 32, by = (cols + 31) / 32;
    if (by > 65535) return cudaErrorNotSupported;
    ctranspose_kernel<R><<<dim3((unsigned)bx, (unsigned)by), 256, 0, s>>>(src, lds, dst, ldd, rows, cols);
    count_launch();
    return cudaGetLastError();
}

template cudaError_t complex_scale<float>(float*, size_t, size_t, size_t, float, float, cudaStream_t);
template cudaError_t complex_scale<double>(double*, size_t, size_t, size_t, double, double, cudaStream_t);
template cudaError_t complex_transpose<float>(float*, size_t, const float*, size_t, size_t, size_t, cudaStream_t);
template cudaError_t complex_transpose<double>(double*, size_t, const double*, size_t, size_t, size_t, cudaStream_t);

// ta / tb: 0 = NoTrans, 1 = Trans, 2 = ConjTrans.  Pointers are to the real parts of the first
// elements; leading dimensions count complex elements.
template <typename R>
cudaError_t cgemm_colmajor(int ta, int tb, size_t M, size_t N, size_t K, R ar, R ai, const R* A, size_t lda,
                           const R* B, size_t ldb, R br, R bi, R* C, size_t ldc, cudaStream_t s, int tri)
{
    if (M == 0 || N == 0) return cudaSuccess;
    if (K == 0 || (ar == R(0) && ai == R(0))) {
        if (tri != TRI_FULL) return complex_tri_scale<R>(tri == TRI_LOWER, N, br, bi, C, ldc, false, s);
        return complex_scale<R>(C, ldc, M, N, br, bi, s);
    }

    constexpr size_t Q = 16 / sizeof(R);
    auto round_up = [](size_t v, size_t q) { return (v + q - 1) / q * q; };
    const size_t lde = round_up(2 * (ta ? K : M), Q);            // A~ is 2M x 2K, or 2K x 2M transposed
    const size_t e_n = lde * 2 * (ta ? M : K);
    const size_t ldp = round_up(N, Q);
    const size_t p_n = tb ? ldp * 2 * K : 0;
    R* ws = nullptr;
    cudaError_t e = ws_alloc(reinterpret_cast<void**>(&ws), (round_up(e_n, 64) + p_n) * sizeof(R) + 256, s);
    if (e != cudaSuccess) return e;
    R* E = ws;
    R* P = ws + round_up(e_n, 64);

    R beta = br;
    if (bi != R(0)) {                       // complex beta: scale first, then accumulate
        e = tri != TRI_FULL ? complex_tri_scale<R>(tri == TRI_LOWER, N, br, bi, C, ldc, false, s)
                            : complex_scale<R>(C, ldc, M, N, br, bi, s);
        beta = R(1);
    }
    if (e == cudaSuccess) {
        if (!ta) expand_a_kernel<R, false><<<grid_for(M * K), 256, 0, s>>>(A, lda, E, lde, M, K, ar, ai, false);
        else     expand_a_kernel<R, true><<<grid_for(M * K), 256, 0, s>>>(A, lda, E, lde, K, M, ar, ai, ta == 2);
        count_launch();
        e = cudaGetLastError();
    }
    if (e == cudaSuccess && tb) {
        planar_b_kernel<R><<<grid_for(N * K), 256, 0, s>>>(B, ldb, P, ldp, N, K, tb == 2);
        count_launch();
        e = cudaGetLastError();
    }
    if (e == cudaSuccess) {
        GemmProblem<R> p;
        p.ta = ta != 0; p.tb = tb != 0;
        p.M = 2 * M; p.N = N; p.K = 2 * K;
        p.alpha = R(1); p.beta = beta;
        p.A = E; p.lda = lde;
        if (tb) { p.B = P; p.ldb = ldp; } else { p.B = B; p.ldb = 2 * ldb; }
        p.C = C; p.ldc = 2 * ldc;
        if (tri != TRI_FULL) p.tri = tri | TRI_PAIRED_ROWS;
        e = gemm_colmajor<R>(p, s);
    }
    const cudaError_t e2 = ws_free(ws, s);
    return e != cudaSuccess ? e : e2;
}

template cudaError_t cgemm_colmajor<float>(int, int, size_t, size_t, size_t, float, float, const float*, size_t, const float*,
                                           size_t, float, float, float*, size_t, cudaStream_t, int);
template cudaError_t cgemm_colmajor<double>(int, int, size_t, size_t, size_t, double, double, const double*, size_t,
                                            const double*, size_t, double, double, double*, size_t, cudaStream_t, int);

}  // namespace cb200
