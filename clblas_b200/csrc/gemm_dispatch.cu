// Tile-config dispatcher: chooses the kernel family for one column-major GEMM from precision,
// transposes, shape and operand alignment.  It stands where the reference has the generated
// gemmSelectKernel<T> decision tree and the shape-triggered GemmSpecialCases
// (src/library/blas/AutoGemm/KernelSelection.py:30-305, src/library/blas/specialCases/
// GemmSpecialCases.cpp:827-952): the reference picks the largest tile that divides M and N and
// pays extra launches otherwise; here every family handles ragged M, N, K in one launch, so the
// questions are (1) can the operands be fetched by TMA (16-byte aligned base addresses and leading
// dimensions) and (2) is it worth giving an operand a better layout first:
//   * an operand TMA cannot address is copied once into an aligned workspace when the product is
//     large enough for the copy to pay (offsets of a few elements, odd leading dimensions);
//   * for SGEMM a K-contiguous operand is transposed on the way, so that large products always run
//     the fastest (N/T) variant of the FFMA kernel;
//   * everything else (small or huge unaligned problems, or when allocation is not allowed) runs
//     the alignment-free kernel in place.
#include "common.h"

#include <algorithm>
#include <cstdlib>

namespace cb200 {

namespace {

thread_local int t_forbid_alloc = 0;

constexpr size_t kMaxRepackBytes = size_t(3) << 30;      // per operand

template <typename T>
cudaError_t degenerate(const GemmProblem<T>& p, cudaStream_t s, bool* handled)
{
    *handled = true;
    if (p.M == 0 || p.N == 0) return cudaSuccess;
    if (p.K == 0 || p.alpha == T(0)) {
        // BLAS semantics: C <- beta*C, A and B are not referenced.
        set_last_kernel("scale");
        if (p.beta == T(1)) return cudaSuccess;
        return launch_scale<T>(p.M, p.N, p.beta, p.C, p.ldc, s);
    }
    *handled = false;
    return cudaSuccess;
}

template <typename T> cudaError_t launch_tma(const GemmProblem<T>& p, cudaStream_t s);
template <> cudaError_t launch_tma<float>(const GemmProblem<float>& p, cudaStream_t s) { return launch_sgemm_ffma_tma(p, s); }
template <> cudaError_t launch_tma<double>(const GemmProblem<double>& p, cudaStream_t s) { return launch_dgemm_mma_tma(p, s); }

template <typename T>
bool tma_addressable(const T* ptr, size_t ld)
{
    return aligned16(ptr) && (ld * sizeof(T)) % 16 == 0;
}

inline cudaError_t try_3xtf32(const GemmProblem<float>& p, cudaStream_t s) { return launch_sgemm_3xtf32(p, s); }
inline cudaError_t try_3xtf32(const GemmProblem<double>&, cudaStream_t) { return cudaErrorNotSupported; }

// What to do with one operand before the product.
enum Fix { KEEP, COPY, TRANSPOSE };

template <typename T>
cudaError_t gemm_any(const GemmProblem<T>& p, cudaStream_t s)
{
    bool handled;
    cudaError_t e = degenerate(p, s, &handled);
    if (handled) return e;
    if (forced_gemm_path() == PATH_SIMT_LDG) return launch_gemm_simt<T>(p, s);
    if (forced_gemm_path() == PATH_3XTF32 && t_forbid_alloc == 0 && p.tri == TRI_FULL) {
        e = try_3xtf32(p, s);
        if (e != cudaErrorNotSupported) return e;
    }

    constexpr bool kFloat = sizeof(T) == 4;
    // stored extents: rows are the contiguous direction
    const size_t a_rows = p.ta ? p.K : p.M, a_cols = p.ta ? p.M : p.K;
    const size_t b_rows = p.tb ? p.N : p.K, b_cols = p.tb ? p.K : p.N;
    const bool okA = tma_addressable(p.A, p.lda), okB = tma_addressable(p.B, p.ldb);

    Fix fa = KEEP, fb = KEEP;
    const bool may_alloc = t_forbid_alloc == 0 && forced_gemm_path() == PATH_AUTO;
    const double work = 2.0 * (double)p.M * (double)p.N * (double)p.K;
    static const double transpose_min_work = [] { const char* v = getenv("CLBLAS_B200_TRANSPOSE_MIN_WORK"); return v ? atof(v) : 3e9; }();
    if (may_alloc && p.K >= 64 && work >= (kFloat ? std::min(transpose_min_work, 1.5e10) : 1.5e10)) {
        // The extra pass over an operand is paid back by the other dimension of C; products below
        // about 2000^3 are too short for the extra launches of a plain copy to pay.  A transposition for SGEMM
        // pays from about 1150^3 on (TFLOP/s, transposed first / in place: N/N 1152^3 35.9 / 31.7, 1536^3 48.2 / 40.6,
        // 4096^3 60.5 / 46.4; T/N 1152^3 33.5 / 27.1; but N/N 1024^3 29.8 / 31.6): the kernels for K-contiguous
        // operands are bound by shared-memory bandwidth and cannot use the 16 x 8 register tile.
        if (work >= 1.5e10) {
            if (!okA && p.N >= 512) fa = COPY;
            if (!okB && p.M >= 512) fb = COPY;
        }
        if (kFloat && work >= transpose_min_work && (work >= 1.5e10 || (okA && okB && p.K >= 1024))) {
            if (p.ta && p.N >= 1024 && p.M >= 256) fa = TRANSPOSE;      // K-contiguous A -> M-contiguous
            if (!p.tb && p.M >= 1024 && p.N >= 256) fb = TRANSPOSE;     // K-contiguous B -> N-contiguous
        }
        if (fa != KEEP && a_rows * a_cols * sizeof(T) > kMaxRepackBytes) fa = KEEP;
        if (fb != KEEP && b_rows * b_cols * sizeof(T) > kMaxRepackBytes) fb = KEEP;
    }
    if ((fa == KEEP && !okA) || (fb == KEEP && !okB)) return launch_gemm_simt<T>(p, s);
    if (fa == KEEP && fb == KEEP) {
        e = launch_tma<T>(p, s);
        return e == cudaErrorNotSupported ? launch_gemm_simt<T>(p, s) : e;
    }

    // ---- repack into one stream-ordered workspace, multiply, release
    constexpr size_t Q = 16 / sizeof(T);
    auto round_up = [](size_t v, size_t q) { return (v + q - 1) / q * q; };
    const size_t a_ld = fa == TRANSPOSE ? round_up(a_cols, Q) : round_up(a_rows, Q);
    const size_t a_n = fa == KEEP ? 0 : a_ld * (fa == TRANSPOSE ? a_rows : a_cols);
    const size_t b_ld = fb == TRANSPOSE ? round_up(b_cols, Q) : round_up(b_rows, Q);
    // A * A^T (rank-k update): both operands are one stored matrix, repacked once
    const bool same = fa != KEEP && fa == fb && p.A == p.B && p.lda == p.ldb && a_rows == b_rows && a_cols == b_cols;
    const size_t b_n = fb == KEEP || same ? 0 : b_ld * (fb == TRANSPOSE ? b_rows : b_cols);
    T* ws = nullptr;
    e = ws_alloc(reinterpret_cast<void**>(&ws), (round_up(a_n, 64) + b_n) * sizeof(T) + 256, s);
    if (e != cudaSuccess) {
        cudaGetLastError();
        if (okA && okB) {
            e = launch_tma<T>(p, s);
            return e == cudaErrorNotSupported ? launch_gemm_simt<T>(p, s) : e;
        }
        return launch_gemm_simt<T>(p, s);
    }
    GemmProblem<T> q = p;
    if (fa != KEEP) {
        e = launch_repack<T>(ws, a_ld, p.A, p.lda, a_rows, a_cols, fa == TRANSPOSE, s);
        q.A = ws; q.lda = a_ld;
        if (fa == TRANSPOSE) q.ta = !p.ta;
    }
    if (same) {
        q.B = ws; q.ldb = a_ld;
        if (fb == TRANSPOSE) q.tb = !p.tb;
    } else if (e == cudaSuccess && fb != KEEP) {
        T* wb = ws + round_up(a_n, 64);
        e = launch_repack<T>(wb, b_ld, p.B, p.ldb, b_rows, b_cols, fb == TRANSPOSE, s);
        q.B = wb; q.ldb = b_ld;
        if (fb == TRANSPOSE) q.tb = !p.tb;
    }
    if (e == cudaSuccess) {
        e = launch_tma<T>(q, s);
        if (e == cudaErrorNotSupported) e = launch_gemm_simt<T>(q, s);
    }
    const cudaError_t e2 = ws_free(ws, s);
    return e != cudaSuccess ? e : e2;
}

}  // namespace

bool gemm_may_allocate() { return t_forbid_alloc == 0 && forced_gemm_path() == PATH_AUTO; }

ScopedNoAlloc::ScopedNoAlloc() { ++t_forbid_alloc; }
ScopedNoAlloc::~ScopedNoAlloc() { --t_forbid_alloc; }

template <>
cudaError_t gemm_colmajor<float>(const GemmProblem<float>& p, cudaStream_t s) { return gemm_any<float>(p, s); }

template <>
cudaError_t gemm_colmajor<double>(const GemmProblem<double>& p, cudaStream_t s) { return gemm_any<double>(p, s); }

}  // namespace cb200
