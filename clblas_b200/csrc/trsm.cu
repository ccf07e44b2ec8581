// Blocked triangular solve: op(A) X = alpha B (Left) or X op(A) = alpha B (Right), X over B.
//
// Same two ingredients as the reference's DTRSM (src/library/blas/xtrsm.cc:1136-1507): explicit
// inverses of the NB x NB diagonal blocks of A, and GEMM for everything else.  Differences:
//  * one kernel launch inverts all diagonal blocks (the reference needs a diag_dtrtri launch plus
//    six triple_dgemm_update launches, xtrsm.cc:790-1134);
//  * the substitution is recursive (solve first half, one large-K GEMM update of the second half,
//    solve second half) instead of a rank-NB update per block step, so the updates are large GEMMs;
//  * X is produced in place: only an NB-wide panel is staged, not an M x N copy of B
//    (the reference allocates X = M x N and copies it back, xtrsm.cc:1183-1192, :1480-1497);
//  * the same code serves float (the reference's STRSM goes through its legacy generated kernels,
//    src/library/blas/functor/functor_xtrsm.cc:130-152) and double.
// Only the referenced triangle of A is ever loaded; a unit diagonal is never loaded.
#include "common.h"
#include "tma_pipeline.cuh"

#include <algorithm>
#include <cstdlib>
#include <mutex>

namespace cb200 {

namespace {

constexpr int NB = 128;           // order of the inverted diagonal blocks
constexpr int TRTRI_THREADS = 512;

// Inverts the NB x NB diagonal blocks b_first, b_first + 1, ... (one per CTA) of the triangular matrix A
// (order n) into inv[b] (dense NB x NB, column-major, ld = NB, zeros outside the triangle).  Rows/columns
// of the last block beyond n are completed with the identity.
//
// The block is held in shared memory as a lower-triangular L (an upper-triangular block is loaded
// transposed and the result stored transposed).  X = L^-1 lives in registers, 32 entries per
// thread, and is computed by right-looking forward substitution on the identity:
//   for k: X[k,:] /= L[k,k];  X[i,:] -= L[i,k] * X[k,:]  for all i > k,
// one barrier per k; row k travels through a double-buffered shared row.
template <typename T>
__global__ void __launch_bounds__(TRTRI_THREADS)
trtri_diag_kernel(const T* __restrict__ A, size_t lda, size_t n, bool lower, bool unit, T* __restrict__ inv, unsigned b_first)
{
    extern __shared__ __align__(16) unsigned char smem_raw[];
    T* Ls = reinterpret_cast<T*>(smem_raw);                 // Ls[k*NB + i] = L[i][k]
    T* rowbuf = Ls + NB * NB;                               // 2 x NB
    pdl_launch_dependents();
    pdl_wait();                                             // A may be the result of the kernel before this one

    const size_t b = (size_t)b_first + blockIdx.x;
    const size_t r0 = b * NB;
    const int nv = (n - r0 < (size_t)NB) ? (int)(n - r0) : NB;   // valid order of this block
    const T* Ab = A + r0 + r0 * lda;
    const int t = threadIdx.x;

    for (int e = t; e < NB * NB; e += TRTRI_THREADS) {
        const int i = e % NB, k = e / NB;                   // L[i][k], i >= k is the triangle
        T v = T(0);
        if (i == k) {
            v = (i < nv && !unit) ? Ab[(size_t)i + (size_t)i * lda] : T(1);
        } else if (i > k && i < nv) {
            v = lower ? Ab[(size_t)i + (size_t)k * lda] : Ab[(size_t)k + (size_t)i * lda];
        }
        Ls[k * NB + i] = v;
    }

    // thread (tr, tc) owns X[i][j], i = tr + 16*ii (ii < 8), j = tc + 32*jj (jj < 4)
    const int tc = t % 32, tr = t / 32;
    T x[8][4];
#pragma unroll
    for (int ii = 0; ii < 8; ii++)
#pragma unroll
        for (int jj = 0; jj < 4; jj++) x[ii][jj] = (tr + 16 * ii == tc + 32 * jj) ? T(1) : T(0);
    __syncthreads();

    // k = 16*kb + kk: row k belongs to the threads with tr == kk, register row kb (kept a
    // compile-time index so that x stays in registers).
#pragma unroll
    for (int kb = 0; kb < NB / 16; kb++) {
#pragma unroll 1
        for (int kk = 0; kk < 16; kk++) {
            const int k = kb * 16 + kk;
            // Row k of X is zero beyond column k, so only the column groups jj <= k / 32 = kb / 2 take part
            // (a compile-time bound: kb is an unrolled index).
            const int jmax = kb >> 1;
            T* rb = rowbuf + (k & 1) * NB;
            if (tr == kk) {
                const T rd = T(1) / Ls[k * NB + k];
#pragma unroll
                for (int jj = 0; jj < 4; jj++) {
                    if (jj > jmax) continue;
                    x[kb][jj] = x[kb][jj] * rd;
                    rb[tc + 32 * jj] = x[kb][jj];
                }
            }
            __syncthreads();
            T xr[4];
#pragma unroll
            for (int jj = 0; jj < 4; jj++) xr[jj] = (jj > jmax) ? T(0) : rb[tc + 32 * jj];
#pragma unroll
            for (int ii = 0; ii < 8; ii++) {
                if (ii < kb) continue;                       // rows above the current block row are final
                if (ii == kb && tr <= kk) continue;          // rows up to k inside the block row are final
                const T l = Ls[k * NB + tr + 16 * ii];
#pragma unroll
                for (int jj = 0; jj < 4; jj++) {
                    if (jj > jmax) continue;
                    x[ii][jj] = fma(-l, xr[jj], x[ii][jj]);
                }
            }
        }
    }

    T* out = inv + b * (size_t)(NB * NB);
#pragma unroll
    for (int ii = 0; ii < 8; ii++)
#pragma unroll
        for (int jj = 0; jj < 4; jj++) {
            const int i = tr + 16 * ii, j = tc + 32 * jj;
            if (lower) out[i + j * NB] = x[ii][jj]; else out[j + i * NB] = x[ii][jj];
        }
}

template <typename T>
struct TrsmCtx {
    bool right, lower, trans, eff_lower;
    bool unit = false;
    size_t M, N, n;              // n = order of A
    const T* A; size_t lda;
    T* B; size_t ldb;
    T* inv;                      // NB*NB per diagonal block
    T* tmp;                      // staging panel for one leaf
    cudaStream_t s;
    TrsmPanelGate* gate = nullptr;   // set when columns of A are still arriving (see common.h)
    bool fused = false;              // ranges of up to four diagonal blocks go to the fused kernel (FP64, Left, few columns)
};

// The end of the recursion for double precision, Left side, few right-hand sides: one launch solves the whole range.
inline cudaError_t solve_fused(const TrsmCtx<double>& c, size_t b0, size_t b1, double alpha)
{
    const size_t nblk = (c.n + NB - 1) / NB;
    return launch_dtrsm_diag_fused(c.trans, c.eff_lower, c.A, c.lda, c.n, c.inv, nblk, c.B, c.ldb, c.N, alpha, b0, b1, c.s);
}
inline cudaError_t solve_fused(const TrsmCtx<float>&, size_t, size_t, float) { return cudaErrorNotSupported; }

constexpr size_t trtri_smem(size_t elem) { return (size_t)(NB * NB + 2 * NB) * elem; }

template <typename T>
cudaError_t trtri_prepare()
{
    // The opt-in to more than 48 KB of dynamic shared memory is a per-device function attribute.
    static DeviceOnce once[2];
    return once[sizeof(T) == 8].run([] {
        return cudaFuncSetAttribute(trtri_diag_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)trtri_smem(sizeof(T)));
    });
}

// Inverts the diagonal blocks [b0, b1) of c.A into c.inv.
template <typename T>
cudaError_t invert_blocks(const TrsmCtx<T>& c, size_t b0, size_t b1)
{
    if (b1 <= b0) return cudaSuccess;
    const cudaError_t e = launch_pdl(trtri_diag_kernel<T>, dim3((unsigned)(b1 - b0)), dim3(TRTRI_THREADS), trtri_smem(sizeof(T)), c.s,
                                     c.A, c.lda, c.n, c.lower, c.unit, c.inv, (unsigned)b0);
    count_launch();
    return e;
}

// Before an operation that reads columns [c0, c1) of the stored A: with a gate, orders the stream after
// the arrival of every panel that holds one of them and has not been waited for yet, and inverts the
// diagonal blocks of those panels.  Without a gate everything is in place already.
template <typename T>
cudaError_t need_columns(const TrsmCtx<T>& c, size_t c0, size_t c1)
{
    TrsmPanelGate* g = c.gate;
    if (g == nullptr) return cudaSuccess;
    for (size_t p = 0; p + 1 < g->bounds.size(); p++) {
        const size_t p0 = g->bounds[p], p1 = g->bounds[p + 1];
        if (p1 <= c0 || p0 >= c1 || g->waited[p]) continue;
        cudaError_t e = cudaStreamWaitEvent(c.s, g->ready[p], 0);
        if (e != cudaSuccess) return e;
        g->waited[p] = 1;
        if ((e = invert_blocks(c, p0 / NB, (p1 + NB - 1) / NB)) != cudaSuccess) return e;
    }
    return cudaSuccess;
}

template <typename T>
cudaError_t gemm_call(bool ta, bool tb, size_t M, size_t N, size_t K, T alpha, const T* A, size_t lda,
                      const T* B, size_t ldb, T beta, T* C, size_t ldc, cudaStream_t s)
{
    GemmProblem<T> p;
    p.ta = ta; p.tb = tb; p.M = M; p.N = N; p.K = K; p.alpha = alpha; p.A = A; p.lda = lda;
    p.B = B; p.ldb = ldb; p.beta = beta; p.C = C; p.ldc = ldc;
    return gemm_colmajor<T>(p, s);
}

// TMA-staged product whose output aliases one of its inputs (see solve_leaf); NotSupported when the
// operands are not TMA-addressable.  For the FP64 kernel the tile must span all 128 columns when the
// aliased operand is A (Right side), so the narrow-tile variants are excluded there.
inline cudaError_t launch_tma_inplace(const GemmProblem<float>& p, cudaStream_t s)
{
    return launch_sgemm_ffma_tma(p, s, p.C == p.A ? 128 : 0);
}
inline cudaError_t launch_tma_inplace(const GemmProblem<double>& p, cudaStream_t s)
{
    return launch_dgemm_mma_tma(p, s, p.C == p.A ? 128 : 0);
}

// X_b = alpha * op(inv_b) * B_b (Left) or alpha * B_b * op(inv_b) (Right) for diagonal block b.
template <typename T>
cudaError_t solve_leaf(const TrsmCtx<T>& c, size_t b, T alpha)
{
    const size_t r = b * NB, nv = std::min<size_t>(NB, c.n - r);
    const T* invb = c.inv + b * (size_t)(NB * NB);
    cudaError_t e;
    if ((e = need_columns(c, r, r + nv)) != cudaSuccess) return e;
    // In place when the TMA kernels can take the panel: their CTA tile is 128 rows (Left) or 128
    // columns (Right) = the whole block, so each CTA reads exactly the part of B it later overwrites,
    // and reads all of it (every K slab) before its epilogue stores; beta = 0 never reads C.
    {
        T* Bb = c.right ? c.B + r * c.ldb : c.B + r;
        GemmProblem<T> p;
        p.alpha = alpha; p.beta = T(0); p.C = Bb; p.ldc = c.ldb; p.K = nv;
        if (!c.right) { p.ta = c.trans; p.tb = false; p.M = nv; p.N = c.N; p.A = invb; p.lda = NB; p.B = Bb; p.ldb = c.ldb; }
        else          { p.ta = false; p.tb = c.trans; p.M = c.M; p.N = nv; p.A = Bb; p.lda = c.ldb; p.B = invb; p.ldb = NB; }
        e = launch_tma_inplace(p, c.s);
        if (e != cudaErrorNotSupported) return e;
    }
    if (!c.right) {
        T* Bb = c.B + r;
        e = gemm_call<T>(c.trans, false, nv, c.N, nv, alpha, invb, NB, Bb, c.ldb, T(0), c.tmp, nv, c.s);
        if (e != cudaSuccess) return e;
        return cudaMemcpy2DAsync(Bb, c.ldb * sizeof(T), c.tmp, nv * sizeof(T), nv * sizeof(T), c.N,
                                 cudaMemcpyDeviceToDevice, c.s);
    }
    T* Bb = c.B + r * c.ldb;
    e = gemm_call<T>(false, c.trans, c.M, nv, nv, alpha, Bb, c.ldb, invb, NB, T(0), c.tmp, c.M, c.s);
    if (e != cudaSuccess) return e;
    return cudaMemcpy2DAsync(Bb, c.ldb * sizeof(T), c.tmp, c.M * sizeof(T), c.M * sizeof(T), nv,
                             cudaMemcpyDeviceToDevice, c.s);
}

// Solves for the diagonal blocks [b0, b1) of the system; the right-hand side has already been
// updated with every block outside the range that precedes it in substitution order.
template <typename T>
cudaError_t solve_range(const TrsmCtx<T>& c, size_t b0, size_t b1, T alpha)
{
    if (c.fused && b1 - b0 <= (size_t)dtrsm_diag_fused_max_blocks()) {
        cudaError_t ef = need_columns(c, b0 * NB, std::min<size_t>(b1 * NB, c.n));
        if (ef != cudaSuccess) return ef;
        ef = solve_fused(c, b0, b1, alpha);
        if (ef != cudaErrorNotSupported) return ef;
    }
    if (b1 - b0 == 1) return solve_leaf(c, b0, alpha);
    const size_t mid = b0 + (b1 - b0 + 1) / 2;
    const size_t r0 = b0 * NB, r1 = mid * NB, r2 = std::min<size_t>(b1 * NB, c.n);
    const size_t n1 = r1 - r0, n2 = r2 - r1;        // orders of the first / second half
    cudaError_t e;
    // Which half is solved first: the one op(A) couples only to itself.
    const bool first_half_first = (c.eff_lower != c.right);
    if (first_half_first) {
        if ((e = solve_range(c, b0, mid, alpha)) != cudaSuccess) return e;
        if (!c.right) {
            // B2 = alpha*B2 - op(A)[2,1] * X1 ; op(A)[2,1] is A[2,1] or A[1,2]^T
            const T* A21 = c.trans ? c.A + r0 + r1 * c.lda : c.A + r1 + r0 * c.lda;
            if ((e = c.trans ? need_columns(c, r1, r2) : need_columns(c, r0, r1)) != cudaSuccess) return e;
            e = gemm_call<T>(c.trans, false, n2, c.N, n1, T(-1), A21, c.lda, c.B + r0, c.ldb, alpha, c.B + r1, c.ldb, c.s);
        } else {
            // X op(A) = alpha B with op(A) upper: B2 = alpha*B2 - X1 * op(A)[1,2]
            const T* A12 = c.trans ? c.A + r1 + r0 * c.lda : c.A + r0 + r1 * c.lda;
            if ((e = c.trans ? need_columns(c, r0, r1) : need_columns(c, r1, r2)) != cudaSuccess) return e;
            e = gemm_call<T>(false, c.trans, c.M, n2, n1, T(-1), c.B + r0 * c.ldb, c.ldb, A12, c.lda, alpha,
                             c.B + r1 * c.ldb, c.ldb, c.s);
        }
        if (e != cudaSuccess) return e;
        return solve_range(c, mid, b1, T(1));
    }
    if ((e = solve_range(c, mid, b1, alpha)) != cudaSuccess) return e;
    if (!c.right) {
        // op(A) upper: B1 = alpha*B1 - op(A)[1,2] * X2
        const T* A12 = c.trans ? c.A + r1 + r0 * c.lda : c.A + r0 + r1 * c.lda;
        if ((e = c.trans ? need_columns(c, r0, r1) : need_columns(c, r1, r2)) != cudaSuccess) return e;
        e = gemm_call<T>(c.trans, false, n1, c.N, n2, T(-1), A12, c.lda, c.B + r1, c.ldb, alpha, c.B + r0, c.ldb, c.s);
    } else {
        // X op(A) = alpha B with op(A) lower: B1 = alpha*B1 - X2 * op(A)[2,1]
        const T* A21 = c.trans ? c.A + r0 + r1 * c.lda : c.A + r1 + r0 * c.lda;
        if ((e = c.trans ? need_columns(c, r1, r2) : need_columns(c, r0, r1)) != cudaSuccess) return e;
        e = gemm_call<T>(false, c.trans, c.M, n1, n2, T(-1), c.B + r1 * c.ldb, c.ldb, A21, c.lda, alpha,
                         c.B + r0 * c.ldb, c.ldb, c.s);
    }
    if (e != cudaSuccess) return e;
    return solve_range(c, b0, mid, T(1));
}

inline bool fused_applicable(const TrsmCtx<double>& c)
{
    return !c.right && getenv("CLBLAS_B200_NO_TRSM_FUSE") == nullptr && dtrsm_diag_fused_applicable(c.A, c.lda, c.B, c.ldb, c.n, c.N);
}
inline bool fused_applicable(const TrsmCtx<float>&) { return false; }

}  // namespace

template <typename T>
cudaError_t trsm_colmajor(bool right, bool lower, bool trans, bool unit, size_t M, size_t N, T alpha,
                          const T* A, size_t lda, T* B, size_t ldb, cudaStream_t s, TrsmPanelGate* gate)
{
    if (M == 0 || N == 0) return cudaSuccess;
    if (alpha == T(0)) return launch_scale<T>(M, N, T(0), B, ldb, s);   // BLAS: B <- 0, A not referenced

    TrsmCtx<T> c;
    c.right = right; c.lower = lower; c.trans = trans; c.eff_lower = (lower != trans); c.unit = unit;
    c.M = M; c.N = N; c.n = right ? N : M; c.A = A; c.lda = lda; c.B = B; c.ldb = ldb; c.s = s; c.gate = gate;
    const size_t nblk = (c.n + NB - 1) / NB;
    const size_t inv_elems = nblk * (size_t)(NB * NB);
    const size_t tmp_elems = (size_t)NB * (right ? M : N);
    c.fused = fused_applicable(c);

    cudaError_t e = trtri_prepare<T>();
    if (e != cudaSuccess) return e;
    T* ws = nullptr;
    e = ws_alloc(reinterpret_cast<void**>(&ws), (inv_elems + tmp_elems) * sizeof(T), s);
    if (e != cudaSuccess) return e;
    c.inv = ws;
    c.tmp = ws + inv_elems;

    if (gate == nullptr) e = invert_blocks(c, 0, nblk);    // with a gate: panel by panel, as the panels arrive
    if (e == cudaSuccess) e = solve_range<T>(c, 0, nblk, alpha);
    cudaError_t e2 = ws_free(ws, s);
    return e != cudaSuccess ? e : e2;
}

void trsm_release_workspaces() { ws_release_all(); }

// ---------------------------------------------------------------------------------------------
// DTRSM without any allocation: the workspace of the blocked solve (inverted diagonal blocks and
// the staging panel) lives in a file-scope device array instead of coming from cudaMallocAsync.
//
// It is for callers that must not allocate device memory once they are running: a service that
// hands the whole GPU to its own memory pool at start-up, or a control loop with a fixed memory
// budget in which an allocation that synchronises the device or fails is not acceptable.
//
// The array has a fixed, modest size (12 MiB, held by every GPU that loads this library until the
// process exits), which bounds the problem: order of A <= CLBLAS_B200_NOALLOC_MAX_ORDER and the other
// dimension of B <= CLBLAS_B200_NOALLOC_MAX_OTHER.  All calls on a device share the one array: two
// calls whose kernels can overlap on the GPU (different streams without an ordering between them)
// race on it.  Nothing in it has to start from zero -- the inversion kernel writes every entry of
// every inverted block and each leaf product fully overwrites the part of the panel that is read
// back -- so contents left by an earlier call are harmless.
constexpr size_t NOALLOC_MAX_ORDER = CLBLAS_B200_NOALLOC_MAX_ORDER;
constexpr size_t NOALLOC_MAX_OTHER = CLBLAS_B200_NOALLOC_MAX_OTHER;
constexpr size_t NOALLOC_INV_ELEMS = NOALLOC_MAX_ORDER * NB;           // NB*NB per diagonal block
constexpr size_t NOALLOC_TMP_ELEMS = (size_t)NB * NOALLOC_MAX_OTHER;
static __device__ __align__(256) double g_dtrsm_noalloc_scratch[NOALLOC_INV_ELEMS + NOALLOC_TMP_ELEMS];

// In host code the array's name is only a handle; the device address comes from
// cudaGetSymbolAddress, asked once per device with that device current.
static cudaError_t noalloc_scratch_address(double** out)
{
    static std::mutex mu;
    static double* addr[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> lock(mu);
    if (addr[dev] == nullptr) {
        double* p = nullptr;
        e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_dtrsm_noalloc_scratch);
        if (e != cudaSuccess) return e;
        // Everything else a solve can need for the first time on this device is done here as well: the
        // shared-memory opt-in of the inversion kernel and of every GEMM kernel the dispatcher can choose
        // without allocating, each of them loaded (cudaFuncGetAttributes) -- so that no later call, whatever its
        // transposition, width or alignment, has any first-time work left.
        if ((e = trtri_prepare<double>()) != cudaSuccess) return e;
        cudaFuncAttributes fa;
        if ((e = cudaFuncGetAttributes(&fa, trtri_diag_kernel<double>)) != cudaSuccess) return e;
        if ((e = dgemm_prepare_all_kernels()) != cudaSuccess) return e;
        if ((e = dtrsm_diag_fused_prepare_all()) != cudaSuccess) return e;
        addr[dev] = p;
    }
    *out = addr[dev];
    return cudaSuccess;
}

cudaError_t dtrsm_colmajor_noalloc(bool right, bool lower, bool trans, bool unit, size_t M, size_t N, double alpha,
                                   const double* A, size_t lda, double* B, size_t ldb, cudaStream_t s)
{
    if (M == 0 || N == 0) return cudaSuccess;
    const size_t n = right ? N : M, other = right ? M : N;
    if (n > NOALLOC_MAX_ORDER || other > NOALLOC_MAX_OTHER) return cudaErrorMemoryAllocation;
    if (alpha == 0.0) return launch_scale<double>(M, N, 0.0, B, ldb, s);

    double* ws = nullptr;
    cudaError_t e = noalloc_scratch_address(&ws);
    if (e != cudaSuccess) return e;
    ScopedNoAlloc no_alloc;          // the GEMM dispatcher must not repack operands into a workspace here

    TrsmCtx<double> c;
    c.right = right; c.lower = lower; c.trans = trans; c.eff_lower = (lower != trans); c.unit = unit;
    c.M = M; c.N = N; c.n = n; c.A = A; c.lda = lda; c.B = B; c.ldb = ldb; c.s = s;
    c.inv = ws;
    c.tmp = ws + NOALLOC_INV_ELEMS;
    c.fused = fused_applicable(c);
    const size_t nblk = (n + NB - 1) / NB;
    if ((e = invert_blocks(c, 0, nblk)) != cudaSuccess) return e;
    return solve_range<double>(c, 0, nblk, alpha);
}

// ---------------------------------------------------------------------------------------------
// Complex triangular solve (clblasCtrsm / clblasZtrsm, src/clBLAS.h:8132-8151, :8202-8221;
// src/library/blas/xtrsm.cc:1787-1911) on the real machinery above.
//
// With every complex entry a written as the real 2 x 2 block [[re, -im], [im, re]], the complex system
// op(A) X = B with interleaved (re, im) storage of X and B IS the real system A~ X_real = B_real of twice
// the order, and A~ is triangular by 128 x 128 blocks (64 complex rows each).  So the recursion, its GEMM
// updates and the in-place leaf products above run unchanged on A~ (materialised once, strictly
// block-off-diagonal part only) and on B where it lies; only the inversion of the diagonal blocks is
// complex-aware: it inverts the 64 x 64 complex blocks and stores the 2 x 2-block form of the inverses.
// rep(A)^T = rep(A^H), so A^H is the real solver's transposition of rep(A), A^T that of rep(conj A).
// A Right-side solve is the Left-side solve of the transposed system on a transposed copy of B.
namespace {

constexpr int CNB = NB / 2;       // complex rows per diagonal block

template <typename R> struct Pair2;
template <> struct Pair2<float> { using type = float2; };
template <> struct Pair2<double> { using type = double2; };

// One CTA of CNB threads per diagonal block: thread j computes column j of X = L^-1 by forward
// substitution (L = the block, or its transpose when the triangle is the upper one); the block is
// conjugated on load when asked.  inv[b] receives the 128 x 128 real form of the inverse, completed
// with the identity beyond the order n of the matrix.
template <typename R>
__global__ void __launch_bounds__(CNB)
ctrtri_diag_kernel(const R* __restrict__ A, size_t lda, size_t n, bool lower, bool unit, bool conj, R* __restrict__ inv)
{
    using R2 = typename Pair2<R>::type;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    R2* Ls = reinterpret_cast<R2*>(smem_raw);            // Ls[i * CNB + k] = L[i][k]
    R2* Xs = Ls + CNB * CNB;                             // Xs[k * CNB + j] = X[k][j]
    R2* rinv = Xs + CNB * CNB;                           // 1 / L[i][i]

    const size_t b = blockIdx.x, r0 = b * CNB;
    const int nv = (n - r0 < (size_t)CNB) ? (int)(n - r0) : CNB;
    const R* Ab = A + 2 * (r0 + r0 * lda);
    const int t = threadIdx.x;

    for (int e = t; e < CNB * CNB; e += CNB) {
        const int i = e % CNB, k = e / CNB;              // L[i][k]; i >= k is the triangle
        R2 v; v.x = R(0); v.y = R(0);
        if (i == k) {
            v.x = R(1);
            if (i < nv && !unit) v = *reinterpret_cast<const R2*>(Ab + 2 * ((size_t)i + (size_t)i * lda));
        } else if (i > k && i < nv) {
            v = lower ? *reinterpret_cast<const R2*>(Ab + 2 * ((size_t)i + (size_t)k * lda))
                      : *reinterpret_cast<const R2*>(Ab + 2 * ((size_t)k + (size_t)i * lda));
        }
        if (conj) v.y = -v.y;
        Ls[i * CNB + k] = v;
    }
    __syncthreads();
    {
        const R2 d = Ls[t * CNB + t];
        const R den = d.x * d.x + d.y * d.y;
        R2 r; r.x = d.x / den; r.y = -d.y / den;
        rinv[t] = r;
    }
    __syncthreads();

    const int j = t;
    for (int i = 0; i < CNB; i++) {
        R2 x; x.x = R(0); x.y = R(0);
        if (i == j) {
            x = rinv[i];
        } else if (i > j) {
            R sr = R(0), si = R(0);
            for (int k = j; k < i; k++) {
                const R2 l = Ls[i * CNB + k], y = Xs[k * CNB + j];
                sr += l.x * y.x - l.y * y.y;
                si += l.x * y.y + l.y * y.x;
            }
            const R2 q = rinv[i];
            x.x = -(sr * q.x - si * q.y);
            x.y = -(sr * q.y + si * q.x);
        }
        Xs[i * CNB + j] = x;                             // only this thread reads column j back
    }
    __syncthreads();

    R* out = inv + b * (size_t)(NB * NB);
    for (int e = t; e < NB * NB; e += CNB) {
        const int r = e % NB, c = e / NB;
        const int i = r / 2, k = c / 2;
        const R2 v = lower ? Xs[i * CNB + k] : Xs[k * CNB + i];      // inverse of an upper block = transposed result
        const int pr = r & 1, pc = c & 1;
        out[e] = (pr == pc) ? v.x : (pr ? v.y : -v.y);
    }
}

// A~ from the referenced triangle of A, blocks strictly off the block diagonal only (the diagonal blocks
// are used through their inverses).  i runs along the contiguous direction.
template <typename R>
__global__ void __launch_bounds__(256) expand_tri_kernel(const R* __restrict__ A, size_t lda, R* __restrict__ E, size_t lde,
                                                         size_t n, bool lower, bool conj)
{
    using R2 = typename Pair2<R>::type;
    const size_t total = n * n;
    for (size_t e = (size_t)blockIdx.x * 256 + threadIdx.x; e < total; e += (size_t)gridDim.x * 256) {
        const size_t i = e % n, j = e / n;
        const size_t bi = i / CNB, bj = j / CNB;
        if (lower ? bi <= bj : bi >= bj) continue;
        R2 a = *reinterpret_cast<const R2*>(A + 2 * (i + j * lda));
        if (conj) a.y = -a.y;
        R2 c0, c1;
        c0.x = a.x; c0.y = a.y; c1.x = -a.y; c1.y = a.x;
        *reinterpret_cast<R2*>(E + 2 * i + (2 * j) * lde) = c0;
        *reinterpret_cast<R2*>(E + 2 * i + (2 * j + 1) * lde) = c1;
    }
}

template <typename R>
cudaError_t ctrsm_left(bool lower, int op, bool unit, size_t M, size_t N, const R* A, size_t lda, R* B, size_t ldb,
                       cudaStream_t s)
{
    // op: 0 A, 1 A^T, 2 A^H, 3 conj(A)
    const bool conj = (op == 1 || op == 3), rtrans = (op == 1 || op == 2);
    TrsmCtx<R> c;
    c.right = false; c.lower = lower; c.trans = rtrans; c.eff_lower = (lower != rtrans);
    c.M = 2 * M; c.N = N; c.n = 2 * M; c.B = B; c.ldb = 2 * ldb; c.s = s;
    const size_t nblk = (M + CNB - 1) / CNB;
    const size_t inv_elems = nblk * (size_t)(NB * NB);
    const size_t tmp_elems = (size_t)NB * N;
    constexpr size_t Q = 16 / sizeof(R);
    const size_t lde = (2 * M + Q - 1) / Q * Q;
    const size_t e_elems = nblk > 1 ? lde * 2 * M : 0;

    R* ws = nullptr;
    cudaError_t e = ws_alloc(reinterpret_cast<void**>(&ws), (inv_elems + tmp_elems + e_elems) * sizeof(R), s);
    if (e != cudaSuccess) return e;
    c.inv = ws;
    c.tmp = ws + inv_elems;
    R* E = ws + inv_elems + tmp_elems;
    c.A = E; c.lda = lde;
    c.fused = fused_applicable(c);       // the fused kernel reads only blocks off the block diagonal, which is all E holds

    const size_t smem = (size_t)(2 * CNB * CNB + CNB) * 2 * sizeof(R);
    static DeviceOnce once[2];
    e = once[sizeof(R) == 8].run([smem] {
        return cudaFuncSetAttribute(ctrtri_diag_kernel<R>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    });
    if (e != cudaSuccess) { ws_free(ws, s); return e; }
    ctrtri_diag_kernel<R><<<(unsigned)nblk, CNB, smem, s>>>(A, lda, M, lower, unit, conj, c.inv);
    count_launch();
    e = cudaGetLastError();
    if (e == cudaSuccess && nblk > 1) {
        const unsigned blocks = (unsigned)std::min<size_t>((M * M + 255) / 256, (size_t)sm_count() * 16);
        expand_tri_kernel<R><<<blocks, 256, 0, s>>>(A, lda, E, lde, M, lower, conj);
        count_launch();
        e = cudaGetLastError();
    }
    if (e == cudaSuccess) e = solve_range<R>(c, 0, nblk, R(1));
    const cudaError_t e2 = ws_free(ws, s);
    return e != cudaSuccess ? e : e2;
}

}  // namespace

template <typename R>
cudaError_t complex_expand_block_offdiag(const R* A, size_t lda, R* E, size_t lde, size_t n, bool lower, bool conj, cudaStream_t s)
{
    const unsigned blocks = (unsigned)std::min<size_t>((n * n + 255) / 256, (size_t)sm_count() * 16);
    expand_tri_kernel<R><<<blocks, 256, 0, s>>>(A, lda, E, lde, n, lower, conj);
    count_launch();
    return cudaGetLastError();
}
template cudaError_t complex_expand_block_offdiag<float>(const float*, size_t, float*, size_t, size_t, bool, bool, cudaStream_t);
template cudaError_t complex_expand_block_offdiag<double>(const double*, size_t, double*, size_t, size_t, bool, bool, cudaStream_t);

template <typename R>
cudaError_t ctrsm_colmajor(bool right, bool lower, int op, bool unit, size_t M, size_t N, R ar, R ai,
                           const R* A, size_t lda, R* B, size_t ldb, cudaStream_t s)
{
    if (M == 0 || N == 0) return cudaSuccess;
    // B <- alpha*B first (alpha == 0: B <- 0 and A is not referenced), then the solve with alpha = 1
    cudaError_t e = complex_scale<R>(B, ldb, M, N, ar, ai, s);
    if (e != cudaSuccess || (ar == R(0) && ai == R(0))) return e;
    if (!right) return ctrsm_left<R>(lower, op, unit, M, N, A, lda, B, ldb, s);

    // X op(A) = B  <=>  op(A)^T X^T = B^T: (A)^T -> A^T, (A^T)^T -> A, (A^H)^T -> conj(A)
    constexpr size_t Q = 16 / sizeof(R);
    const size_t ldt = (N + Q - 1) / Q * Q;
    R* Bt = nullptr;
    e = ws_alloc(reinterpret_cast<void**>(&Bt), 2 * ldt * M * sizeof(R), s);
    if (e != cudaSuccess) return e;
    e = complex_transpose<R>(Bt, ldt, B, ldb, M, N, s);
    if (e == cudaSuccess) e = ctrsm_left<R>(lower, op == 0 ? 1 : op == 1 ? 0 : 3, unit, N, M, A, lda, Bt, ldt, s);
    if (e == cudaSuccess) e = complex_transpose<R>(B, ldb, Bt, ldt, N, M, s);
    const cudaError_t e2 = ws_free(Bt, s);
    return e != cudaSuccess ? e : e2;
}

template cudaError_t ctrsm_colmajor<float>(bool, bool, int, bool, size_t, size_t, float, float, const float*, size_t, float*,
                                           size_t, cudaStream_t);
template cudaError_t ctrsm_colmajor<double>(bool, bool, int, bool, size_t, size_t, double, double, const double*, size_t,
                                            double*, size_t, cudaStream_t);

template cudaError_t trsm_colmajor<float>(bool, bool, bool, bool, size_t, size_t, float, const float*, size_t,
                                          float*, size_t, cudaStream_t, TrsmPanelGate*);
template cudaError_t trsm_colmajor<double>(bool, bool, bool, bool, size_t, size_t, double, const double*, size_t,
                                           double*, size_t, cudaStream_t, TrsmPanelGate*);

}  // namespace cb200
