// Triangular matrix multiply: B <- alpha * op(A) * B (Left) or alpha * B * op(A) (Right), A triangular.
//
// Replaces clblasStrmm / clblasDtrmm (src/clBLAS.h:7697-7717, :7772-7792; src/library/blas/xtrmm.c:116-180),
// which the reference serves with its run-time generated legacy kernels.  Here it is the companion of
// the blocked TRSM: the same recursion over 128 x 128 diagonal blocks with all the off-diagonal work in
// the GEMM kernels (one large-K product per recursion level), and dense copies of the diagonal
// blocks -- zeros outside the referenced triangle, ones on a unit diagonal -- for the leaves.  Only
// the referenced triangle of A is ever loaded.
#include "common.h"

#include <algorithm>

namespace cb200 {

namespace {

constexpr int NB = 128;

// tri[b] = dense NB x NB copy (column-major, ld = NB) of diagonal block b of the triangular matrix A:
// entries outside the referenced triangle and beyond order n are zero, a unit diagonal is written as 1.
template <typename T>
__global__ void __launch_bounds__(256) tri_blocks_kernel(const T* __restrict__ A, size_t lda, size_t n, bool lower, bool unit,
                                                          T* __restrict__ tri)
{
    const size_t b = blockIdx.x, r0 = b * NB;
    const T* Ab = A + r0 + r0 * lda;
    T* out = tri + b * (size_t)(NB * NB);
    for (int e = threadIdx.x; e < NB * NB; e += 256) {
        const int i = e % NB, j = e / NB;
        T v = T(0);
        if (r0 + i < n && r0 + j < n) {
            if (i == j) v = unit ? T(1) : Ab[(size_t)i + (size_t)j * lda];
            else if (lower ? i > j : i < j) v = Ab[(size_t)i + (size_t)j * lda];
        }
        out[e] = v;
    }
}

template <typename T>
struct TrmmCtx {
    bool right, trans, eff_lower;
    size_t M, N, n;
    const T* A; size_t lda;
    T* B; size_t ldb;
    T* tri;
    T* tmp;
    T alpha;
    cudaStream_t s;
};

template <typename T>
cudaError_t gemm_call(bool ta, bool tb, size_t M, size_t N, size_t K, T alpha, const T* A, size_t lda,
                      const T* B, size_t ldb, T beta, T* C, size_t ldc, cudaStream_t s)
{
    GemmProblem<T> p;
    p.ta = ta; p.tb = tb; p.M = M; p.N = N; p.K = K; p.alpha = alpha; p.A = A; p.lda = lda;
    p.B = B; p.ldb = ldb; p.beta = beta; p.C = C; p.ldc = ldc;
    return gemm_colmajor<T>(p, s);
}

inline cudaError_t launch_tma_inplace(const GemmProblem<float>& p, cudaStream_t s)
{
    return launch_sgemm_ffma_tma(p, s, p.C == p.A ? 128 : 0);
}
inline cudaError_t launch_tma_inplace(const GemmProblem<double>& p, cudaStream_t s)
{
    return launch_dgemm_mma_tma(p, s, p.C == p.A ? 128 : 0);
}

// B_b <- alpha * op(tri_b) * B_b (Left) or alpha * B_b * op(tri_b) (Right).  In place with the TMA
// kernels (a CTA covers the whole 128-row / 128-column block, reads exactly what it overwrites and
// reads all of it before storing); through the staging panel otherwise.
template <typename T>
cudaError_t mul_leaf(const TrmmCtx<T>& c, size_t b)
{
    const size_t r = b * NB, nv = std::min<size_t>(NB, c.n - r);
    const T* tb = c.tri + b * (size_t)(NB * NB);
    T* Bb = c.right ? c.B + r * c.ldb : c.B + r;
    GemmProblem<T> p;
    p.alpha = c.alpha; p.beta = T(0); p.C = Bb; p.ldc = c.ldb; p.K = nv;
    if (!c.right) { p.ta = c.trans; p.tb = false; p.M = nv; p.N = c.N; p.A = tb; p.lda = NB; p.B = Bb; p.ldb = c.ldb; }
    else          { p.ta = false; p.tb = c.trans; p.M = c.M; p.N = nv; p.A = Bb; p.lda = c.ldb; p.B = tb; p.ldb = NB; }
    cudaError_t e = launch_tma_inplace(p, c.s);
    if (e != cudaErrorNotSupported) return e;
    if (!c.right) {
        e = gemm_call<T>(c.trans, false, nv, c.N, nv, c.alpha, tb, NB, Bb, c.ldb, T(0), c.tmp, nv, c.s);
        if (e != cudaSuccess) return e;
        return cudaMemcpy2DAsync(Bb, c.ldb * sizeof(T), c.tmp, nv * sizeof(T), nv * sizeof(T), c.N, cudaMemcpyDeviceToDevice, c.s);
    }
    e = gemm_call<T>(false, c.trans, c.M, nv, nv, c.alpha, Bb, c.ldb, tb, NB, T(0), c.tmp, c.M, c.s);
    if (e != cudaSuccess) return e;
    return cudaMemcpy2DAsync(Bb, c.ldb * sizeof(T), c.tmp, c.M * sizeof(T), c.M * sizeof(T), nv, cudaMemcpyDeviceToDevice, c.s);
}

// Multiplies the part of B that belongs to diagonal blocks [b0, b1).  The half whose new value needs
// the OLD value of the other half is finished first (own block product, then the coupling GEMM),
// before the other half is overwritten.
template <typename T>
cudaError_t mul_range(const TrmmCtx<T>& c, size_t b0, size_t b1)
{
    if (b1 - b0 == 1) return mul_leaf(c, b0);
    const size_t mid = b0 + (b1 - b0 + 1) / 2;
    const size_t r0 = b0 * NB, r1 = mid * NB, r2 = std::min<size_t>(b1 * NB, c.n);
    const size_t n1 = r1 - r0, n2 = r2 - r1;
    cudaError_t e;
    // Left with op(A) lower, or Right with op(A) upper: the SECOND half receives the coupling term.
    const bool second_gets_coupling = (c.eff_lower != c.right);
    if (second_gets_coupling) {
        if ((e = mul_range(c, mid, b1)) != cudaSuccess) return e;
        if (!c.right) {
            // B2 += alpha * op(A)[2,1] * B1
            const T* A21 = c.trans ? c.A + r0 + r1 * c.lda : c.A + r1 + r0 * c.lda;
            e = gemm_call<T>(c.trans, false, n2, c.N, n1, c.alpha, A21, c.lda, c.B + r0, c.ldb, T(1), c.B + r1, c.ldb, c.s);
        } else {
            // B2 += alpha * B1 * op(A)[1,2]
            const T* A12 = c.trans ? c.A + r1 + r0 * c.lda : c.A + r0 + r1 * c.lda;
            e = gemm_call<T>(false, c.trans, c.M, n2, n1, c.alpha, c.B + r0 * c.ldb, c.ldb, A12, c.lda, T(1), c.B + r1 * c.ldb, c.ldb, c.s);
        }
        if (e != cudaSuccess) return e;
        return mul_range(c, b0, mid);
    }
    if ((e = mul_range(c, b0, mid)) != cudaSuccess) return e;
    if (!c.right) {
        // B1 += alpha * op(A)[1,2] * B2
        const T* A12 = c.trans ? c.A + r1 + r0 * c.lda : c.A + r0 + r1 * c.lda;
        e = gemm_call<T>(c.trans, false, n1, c.N, n2, c.alpha, A12, c.lda, c.B + r1, c.ldb, T(1), c.B + r0, c.ldb, c.s);
    } else {
        // B1 += alpha * B2 * op(A)[2,1]
        const T* A21 = c.trans ? c.A + r0 + r1 * c.lda : c.A + r1 + r0 * c.lda;
        e = gemm_call<T>(false, c.trans, c.M, n1, n2, c.alpha, c.B + r1 * c.ldb, c.ldb, A21, c.lda, T(1), c.B + r0 * c.ldb, c.ldb, c.s);
    }
    if (e != cudaSuccess) return e;
    return mul_range(c, mid, b1);
}

}  // namespace

template <typename T>
cudaError_t trmm_colmajor(bool right, bool lower, bool trans, bool unit, size_t M, size_t N, T alpha,
                          const T* A, size_t lda, T* B, size_t ldb, cudaStream_t s)
{
    if (M == 0 || N == 0) return cudaSuccess;
    if (alpha == T(0)) return launch_scale<T>(M, N, T(0), B, ldb, s);

    TrmmCtx<T> c;
    c.right = right; c.trans = trans; c.eff_lower = (lower != trans);
    c.M = M; c.N = N; c.n = right ? N : M; c.A = A; c.lda = lda; c.B = B; c.ldb = ldb; c.alpha = alpha; c.s = s;
    const size_t nblk = (c.n + NB - 1) / NB;
    const size_t tri_elems = nblk * (size_t)(NB * NB), tmp_elems = (size_t)NB * (right ? M : N);
    T* ws = nullptr;
    cudaError_t e = ws_alloc(reinterpret_cast<void**>(&ws), (tri_elems + tmp_elems) * sizeof(T), s);
    if (e != cudaSuccess) return e;
    c.tri = ws;
    c.tmp = ws + tri_elems;
    tri_blocks_kernel<T><<<(unsigned)nblk, 256, 0, s>>>(A, lda, c.n, lower, unit, c.tri);
    count_launch();
    e = cudaGetLastError();
    if (e == cudaSuccess) e = mul_range<T>(c, 0, nblk);
    const cudaError_t e2 = ws_free(ws, s);
    return e != cudaSuccess ? e : e2;
}

// ---------------------------------------------------------------------------------------------
// Complex TRMM (clblasCtrmm / clblasZtrmm, src/clBLAS.h:7839, :7909; src/library/blas/xtrmm.c) on the real
// recursion above, the way the complex TRSM uses the real solver: with every complex entry written as the
// real block [[re, -im], [im, re]], alpha*op(A)*B on interleaved storage IS a real triangular product of twice
// the order whose matrix is triangular by 128 x 128 blocks.  The off-diagonal blocks come from one expansion of
// the referenced triangle, the dense diagonal blocks from a complex-aware copy; rep(A)^T = rep(A^H), so A^H is
// the real recursion's transposition of rep(A) and A^T that of rep(conj A); alpha is applied to B first; a
// Right-side product is the Left-side product of the transposed problem on a transposed copy of B.
namespace {

constexpr int CNB = NB / 2;

template <typename R> struct Pair2;
template <> struct Pair2<float> { using type = float2; };
template <> struct Pair2<double> { using type = double2; };

// tri[b] = 128 x 128 real form of the 64 x 64 complex diagonal block b: zeros outside the referenced triangle
// and beyond the order n, (1, 0) on a unit diagonal, conjugated when asked.
template <typename R>
__global__ void __launch_bounds__(256) ctri_blocks_kernel(const R* __restrict__ A, size_t lda, size_t n, bool lower, bool unit,
                                                           bool conj, R* __restrict__ tri)
{
    using R2 = typename Pair2<R>::type;
    const size_t b = blockIdx.x, r0 = b * CNB;
    const R* Ab = A + 2 * (r0 + r0 * lda);
    R* out = tri + b * (size_t)(NB * NB);
    for (int e = threadIdx.x; e < CNB * CNB; e += 256) {
        const int i = e % CNB, j = e / CNB;
        R2 v; v.x = R(0); v.y = R(0);
        if (r0 + i < n && r0 + j < n) {
            if (i == j) {
                if (unit) v.x = R(1); else v = *reinterpret_cast<const R2*>(Ab + 2 * ((size_t)i + (size_t)j * lda));
            } else if (lower ? i > j : i < j) {
                v = *reinterpret_cast<const R2*>(Ab + 2 * ((size_t)i + (size_t)j * lda));
            }
        }
        if (conj) v.y = -v.y;
        R* o = out + 2 * i + (size_t)(2 * j) * NB;
        o[0] = v.x; o[1] = v.y; o[NB] = -v.y; o[NB + 1] = v.x;
    }
}

template <typename R>
cudaError_t ctrmm_left(bool lower, int op, bool unit, size_t M, size_t N, const R* A, size_t lda, R* B, size_t ldb, cudaStream_t s)
{
    // op: 0 A, 1 A^T, 2 A^H, 3 conj(A)
    const bool conj = (op == 1 || op == 3), rtrans = (op == 1 || op == 2);
    TrmmCtx<R> c;
    c.right = false; c.trans = rtrans; c.eff_lower = (lower != rtrans);
    c.M = 2 * M; c.N = N; c.n = 2 * M; c.B = B; c.ldb = 2 * ldb; c.alpha = R(1); c.s = s;
    const size_t nblk = (M + CNB - 1) / CNB;
    const size_t tri_elems = nblk * (size_t)(NB * NB), tmp_elems = (size_t)NB * N;
    constexpr size_t Q = 16 / sizeof(R);
    const size_t lde = (2 * M + Q - 1) / Q * Q;
    const size_t e_elems = nblk > 1 ? lde * 2 * M : 0;
    R* ws = nullptr;
    cudaError_t e = ws_alloc(reinterpret_cast<void**>(&ws), (tri_elems + tmp_elems + e_elems) * sizeof(R), s);
    if (e != cudaSuccess) return e;
    c.tri = ws;
    c.tmp = ws + tri_elems;
    R* E = ws + tri_elems + tmp_elems;
    c.A = E; c.lda = lde;
    ctri_blocks_kernel<R><<<(unsigned)nblk, 256, 0, s>>>(A, lda, M, lower, unit, conj, c.tri);
    count_launch();
    e = cudaGetLastError();
    if (e == cudaSuccess && nblk > 1) e = complex_expand_block_offdiag<R>(A, lda, E, lde, M, lower, conj, s);
    if (e == cudaSuccess) e = mul_range<R>(c, 0, nblk);
    const cudaError_t e2 = ws_free(ws, s);
    return e != cudaSuccess ? e : e2;
}

}  // namespace

template <typename R>
cudaError_t ctrmm_colmajor(bool right, bool lower, int op, bool unit, size_t M, size_t N, R ar, R ai,
                           const R* A, size_t lda, R* B, size_t ldb, cudaStream_t s)
{
    if (M == 0 || N == 0) return cudaSuccess;
    // B <- alpha*B first (alpha == 0: B <- 0 and A is not referenced), then the product with alpha = 1
    cudaError_t e = complex_scale<R>(B, ldb, M, N, ar, ai, s);
    if (e != cudaSuccess || (ar == R(0) && ai == R(0))) return e;
    if (!right) return ctrmm_left<R>(lower, op, unit, M, N, A, lda, B, ldb, s);

    // B op(A) = (op(A)^T B^T)^T: (A)^T -> A^T, (A^T)^T -> A, (A^H)^T -> conj(A)
    constexpr size_t Q = 16 / sizeof(R);
    const size_t ldt = (N + Q - 1) / Q * Q;
    R* Bt = nullptr;
    e = ws_alloc(reinterpret_cast<void**>(&Bt), 2 * ldt * M * sizeof(R), s);
    if (e != cudaSuccess) return e;
    e = complex_transpose<R>(Bt, ldt, B, ldb, M, N, s);
    if (e == cudaSuccess) e = ctrmm_left<R>(lower, op == 0 ? 1 : op == 1 ? 0 : 3, unit, N, M, A, lda, Bt, ldt, s);
    if (e == cudaSuccess) e = complex_transpose<R>(B, ldb, Bt, ldt, N, M, s);
    const cudaError_t e2 = ws_free(Bt, s);
    return e != cudaSuccess ? e : e2;
}

template cudaError_t ctrmm_colmajor<float>(bool, bool, int, bool, size_t, size_t, float, float, const float*, size_t, float*, size_t,
                                           cudaStream_t);
template cudaError_t ctrmm_colmajor<double>(bool, bool, int, bool, size_t, size_t, double, double, const double*, size_t, double*,
                                            size_t, cudaStream_t);

template cudaError_t trmm_colmajor<float>(bool, bool, bool, bool, size_t, size_t, float, const float*, size_t, float*, size_t, cudaStream_t);
template cudaError_t trmm_colmajor<double>(bool, bool, bool, bool, size_t, size_t, double, const double*, size_t, double*, size_t, cudaStream_t);

}  // namespace cb200
