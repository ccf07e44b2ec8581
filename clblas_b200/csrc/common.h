// Internal declarations shared by the host layer and the kernel translation units.
#pragma once

#include <cuda_runtime.h>
#include <atomic>
#include <cstddef>
#include <cstdint>
#include <functional>
#include <vector>

#include "../../include/clblas_b200.h"

namespace cb200 {

// Column-major GEMM problem after the front end has normalised order/ConjTrans
// (row-major calls arrive here with operands swapped, as in the reference's
// force_gemm_column_major, src/library/blas/xgemm.cc:40-61).
// ta / tb: op(X) = X^T when true.  Pointers already include the element offsets.
template <typename T>
struct GemmProblem {
    bool ta, tb;
    size_t M, N, K;
    T alpha;
    const T* A; size_t lda;
    const T* B; size_t ldb;
    T beta;
    T* C; size_t ldc;
    // 0: all of C; TRI_LOWER / TRI_UPPER: only entries with row >= col / row <= col are computed and
    // stored (SYRK); tiles entirely outside the triangle exit at once, the others mask their stores.
    int tri = 0;
};

// TRI_PAIRED_ROWS (or-ed in): rows 2i and 2i+1 of C both belong to row i of the triangle -- a complex matrix
// seen as a real one with interleaved (re, im) rows.
enum { TRI_FULL = 0, TRI_LOWER = 1, TRI_UPPER = 2, TRI_PAIRED_ROWS = 4 };

// true when no entry of the bm x bn tile at (m0, n0) lies in the triangle
__host__ __device__ inline bool tri_tile_outside(int tri, size_t m0, size_t bm, size_t n0, size_t bn)
{
    const int sh = (tri >> 2) & 1, kind = tri & 3;
    const size_t r0 = m0 >> sh, r1 = (m0 + bm - 1) >> sh;
    return kind == TRI_LOWER ? r1 < n0 : kind == TRI_UPPER ? n0 + bn - 1 < r0 : false;
}
// true when every entry of the tile lies in the triangle (no masking needed)
__host__ __device__ inline bool tri_tile_inside(int tri, size_t m0, size_t bm, size_t n0, size_t bn)
{
    const int sh = (tri >> 2) & 1, kind = tri & 3;
    const size_t r0 = m0 >> sh, r1 = (m0 + bm - 1) >> sh;
    return kind == TRI_LOWER ? r0 >= n0 + bn - 1 : kind == TRI_UPPER ? n0 >= r1 : true;
}
__host__ __device__ inline bool tri_masked(int tri, size_t row, size_t col)
{
    const int sh = (tri >> 2) & 1, kind = tri & 3;
    const size_t r = row >> sh;
    return kind == TRI_LOWER ? r < col : kind == TRI_UPPER ? r > col : false;
}

// Triangular updates (SYRK, HERK) handed out stream-K fashion: only the 128 x 128 tiles that touch the triangle are
// enumerated, column of tiles by column of tiles.  Rows of tile column tn that take part: [lo, hi).
__host__ __device__ inline void tri_column_rows(int tri, unsigned tilesM, unsigned tn, unsigned& lo, unsigned& hi)
{
    const int sh = (tri >> 2) & 1, kind = tri & 3;
    const size_t n0 = (size_t)tn * 128;
    lo = 0; hi = tilesM;
    if (kind == TRI_LOWER) {            // tile row tm takes part when its last row, (tm*128 + 127) >> sh, reaches column n0
        const size_t lo_t = (n0 << sh) / 128;
        lo = (unsigned)(lo_t < tilesM ? lo_t : tilesM);
    } else if (kind == TRI_UPPER) {     // ... when its first row, (tm*128) >> sh, is not beyond column n0 + 127
        const size_t hi_t = (((n0 + 128) << sh) - 1) / 128 + 1;
        hi = (unsigned)(hi_t < tilesM ? hi_t : tilesM);
    }
}
// tile number t of that enumeration -> (tm, tn)
__host__ __device__ inline void tri_tile_coords(int tri, unsigned t, unsigned tilesM, unsigned tilesN, unsigned& tm, unsigned& tn)
{
    unsigned before = 0;
    for (unsigned c = 0; c < tilesN; c++) {
        unsigned lo, hi;
        tri_column_rows(tri, tilesM, c, lo, hi);
        if (t < before + (hi - lo)) { tn = c; tm = lo + (t - before); return; }
        before += hi - lo;
    }
    tn = tilesN - 1; tm = tilesM - 1;           // not reached: t is below the number of tiles the host counted
}
// number of 128 x 128 tiles of a matrix of tilesM x tilesN tiles that touch the triangle (all of them for TRI_FULL)
inline size_t tri_tile_count(int tri, size_t tilesM, size_t tilesN)
{
    if ((tri & 3) == TRI_FULL) return tilesM * tilesN;
    size_t n = 0;
    for (size_t c = 0; c < tilesN; c++) {
        unsigned lo, hi;
        tri_column_rows(tri, (unsigned)tilesM, (unsigned)c, lo, hi);
        n += hi - lo;
    }
    return n;
}

// Kernel families (reported by clblasB200LastGemmKernel).
enum GemmPath { PATH_AUTO = 0, PATH_SIMT_LDG = 1, PATH_TMA_ONE_CTA = 2, PATH_TMA_TWO_CTAS = 3, PATH_3XTF32 = 4 };

// Optional SGEMM on tcgen05 tensor cores with the 3xTF32 operand split (opt-in, PATH_3XTF32).
cudaError_t launch_sgemm_3xtf32(const GemmProblem<float>& p, cudaStream_t s);
unsigned sgemm_3xtf32_fault_flag();

void count_launch(unsigned n = 1);
void set_last_kernel(const char* name);
// Instantiation and mode of the kernel a GEMM ran (reported by clblasB200LastGemmVariant); the string is copied.
void set_last_variant(const char* name);
int forced_gemm_path();

// Scales C by beta (beta == 0 stores zeros without reading C).  Used for K == 0 and alpha == 0.
template <typename T>
cudaError_t launch_scale(size_t M, size_t N, T beta, T* C, size_t ldc, cudaStream_t s);

// Alignment-free path: predicated, coalesced LDG -> shared -> register-blocked FMA.
template <typename T>
cudaError_t launch_gemm_simt(const GemmProblem<T>& p, cudaStream_t s);

// TMA-staged paths (need 16-byte aligned bases and leading dimensions); return
// cudaErrorNotSupported when the problem does not meet their requirements.
// min_bn: 0 = choose the tile width from the shape; 128 = never use the narrow-tile variants.
cudaError_t launch_dgemm_mma_tma(const GemmProblem<double>& p, cudaStream_t s, int min_bn = 0);
cudaError_t launch_sgemm_ffma_tma(const GemmProblem<float>& p, cudaStream_t s, int min_bn = 0);

// Copies (or transposes) a rows x cols column-major operand into an aligned workspace.
template <typename T>
cudaError_t launch_repack(T* dst, size_t ldd, const T* src, size_t lds, size_t rows, size_t cols, bool transpose,
                          cudaStream_t s);

// While one of these is alive on a thread, gemm_colmajor never allocates (no operand repacking).
struct ScopedNoAlloc {
    ScopedNoAlloc();
    ~ScopedNoAlloc();
};

// False while a ScopedNoAlloc is alive on the calling thread or a kernel family is forced.
bool gemm_may_allocate();

// Dispatcher keyed on precision, transposes, shape and alignment.
template <typename T>
cudaError_t gemm_colmajor(const GemmProblem<T>& p, cudaStream_t s);

// Complex GEMM on the real kernels (cgemm.cu).  ta / tb: 0 NoTrans, 1 Trans, 2 ConjTrans; pointers are to
// the real part of the first element, leading dimensions count complex elements.
// tri: TRI_FULL, or TRI_LOWER / TRI_UPPER to compute and store only that triangle of the (square) complex C.
template <typename R>
cudaError_t cgemm_colmajor(int ta, int tb, size_t M, size_t N, size_t K, R ar, R ai, const R* A, size_t lda,
                           const R* B, size_t ldb, R br, R bi, R* C, size_t ldc, cudaStream_t s, int tri = TRI_FULL);

// C <- beta*C on one triangle of an N x N complex matrix; imaginary parts of the diagonal set to zero when asked.
template <typename R>
cudaError_t complex_tri_scale(bool lower, size_t N, R br, R bi, R* C, size_t ldc, bool zero_diag_imag, cudaStream_t s);

// Complex symmetric / Hermitian rank-k and rank-2k updates and symmetric / Hermitian products (csyrk.cu).
// op: 0 NoTrans, 1 Trans (SYRK/SYR2K), 2 ConjTrans (HERK/HER2K).
template <typename R>
cudaError_t csyrk_colmajor(bool herm, bool lower, int op, size_t N, size_t K, R ar, R ai, const R* A, size_t lda,
                           R br, R bi, R* C, size_t ldc, cudaStream_t s);
template <typename R>
cudaError_t csyr2k_colmajor(bool herm, bool lower, int op, size_t N, size_t K, R ar, R ai, const R* A, size_t lda,
                            const R* B, size_t ldb, R br, R bi, R* C, size_t ldc, cudaStream_t s);
template <typename R>
cudaError_t csymm_colmajor(bool herm, bool right, bool lower, size_t M, size_t N, R ar, R ai, const R* A, size_t lda,
                           const R* B, size_t ldb, R br, R bi, R* C, size_t ldc, cudaStream_t s);

// C <- beta*C on an M x N complex matrix (beta == 0 stores zeros without reading); dst = src^T for complex matrices.
template <typename R>
cudaError_t complex_scale(R* C, size_t ldc, size_t M, size_t N, R br, R bi, cudaStream_t s);
template <typename R>
cudaError_t complex_transpose(R* dst, size_t ldd, const R* src, size_t lds, size_t rows, size_t cols, cudaStream_t s);

// Complex triangular solve (trsm.cu): op 0 NoTrans, 1 Trans, 2 ConjTrans; B (M x N complex) overwritten by X.
template <typename R>
cudaError_t ctrsm_colmajor(bool right, bool lower, int op, bool unit, size_t M, size_t N, R ar, R ai,
                           const R* A, size_t lda, R* B, size_t ldb, cudaStream_t s);

// GEMM on host matrices with uploads, products and downloads overlapped (host_gemm.cu); ordered on `user`.
template <typename T>
cudaError_t gemm_host_colmajor(bool ta, bool tb, size_t M, size_t N, size_t K, T alpha, const T* hA, size_t lda,
                               const T* hB, size_t ldb, T beta, T* hC, size_t ldc, cudaStream_t user);
template <typename T>
cudaError_t trsm_host_colmajor(bool right, bool lower, bool trans, bool unit, size_t M, size_t N, T alpha,
                               const T* hA, size_t lda, T* hB, size_t ldb, cudaStream_t user);
void host_pipeline_release();

// 2 x 2-block real form of the referenced triangle of a complex triangular matrix, blocks of 64 complex rows
// strictly off the block diagonal only (trsm.cu); complex TRMM (trmm.cu), op as for ctrsm_colmajor.
template <typename R>
cudaError_t complex_expand_block_offdiag(const R* A, size_t lda, R* E, size_t lde, size_t n, bool lower, bool conj, cudaStream_t s);
template <typename R>
cudaError_t ctrmm_colmajor(bool right, bool lower, int op, bool unit, size_t M, size_t N, R ar, R ai,
                           const R* A, size_t lda, R* B, size_t ldb, cudaStream_t s);

// Columns of the stored triangular matrix that arrive while the solve is already running (a broadcast
// in column panels): panel p = columns [bounds[p], bounds[p+1]), complete once ready[p] has fired.  Every
// step of the solve waits, on its stream, for the panels it reads and has not waited for yet; the
// diagonal blocks of a panel are inverted when the panel is first needed.  Boundaries other than the
// last one are multiples of 128 (the order of the inverted blocks).
struct TrsmPanelGate {
    std::vector<size_t> bounds;
    std::vector<cudaEvent_t> ready;
    std::vector<char> waited;
};

// Blocked triangular solve on a column-major problem (B overwritten by X).  gate == nullptr: all of A is
// in place when the call is made.
template <typename T>
cudaError_t trsm_colmajor(bool right, bool lower, bool trans, bool unit, size_t M, size_t N, T alpha,
                          const T* A, size_t lda, T* B, size_t ldb, cudaStream_t s, TrsmPanelGate* gate = nullptr);
void trsm_release_workspaces();

// Triangular matrix multiply on a column-major problem (B overwritten by alpha*op(A)*B or alpha*B*op(A)).
template <typename T>
cudaError_t trmm_colmajor(bool right, bool lower, bool trans, bool unit, size_t M, size_t N, T alpha,
                          const T* A, size_t lda, T* B, size_t ldb, cudaStream_t s);

// Symmetric rank-k update of one triangle of C (column-major): C <- alpha*op(A)*op(A)^T + beta*C,
// op(A) = A (N x K) or A^T (A stored K x N).
template <typename T>
cudaError_t syrk_colmajor(bool lower, bool trans, size_t N, size_t K, T alpha, const T* A, size_t lda, T beta,
                          T* C, size_t ldc, cudaStream_t s);

// Symmetric rank-2k update of one triangle of C: C <- alpha*op(A)*op(B)^T + alpha*op(B)*op(A)^T + beta*C.
template <typename T>
cudaError_t syr2k_colmajor(bool lower, bool trans, size_t N, size_t K, T alpha, const T* A, size_t lda, const T* B,
                           size_t ldb, T beta, T* C, size_t ldc, cudaStream_t s);

// C <- alpha*A*B + beta*C (A symmetric M x M) or alpha*B*A + beta*C (right; A symmetric N x N); only the
// `lower` / upper triangle of A is read.
template <typename T>
cudaError_t symm_colmajor(bool right, bool lower, size_t M, size_t N, T alpha, const T* A, size_t lda, const T* B, size_t ldb,
                          T beta, T* C, size_t ldc, cudaStream_t s);

// Multi-GPU forms (sharded.cu).  ShardComm: one rank's end of a communicator (clblasB200Comm).
struct ShardComm;
template <typename T>
cudaError_t gemm_sharded_colmajor(ShardComm* c, int root, const GemmProblem<T>& p, cudaStream_t s);
template <typename T>
cudaError_t trsm_sharded_colmajor(ShardComm* c, int root, bool right, bool lower, bool trans, bool unit, size_t M, size_t N,
                                  T alpha, T* A, size_t lda, T* B, size_t ldb, cudaStream_t s);
// One process, several queues (possibly on several devices): stripe q of N runs on queues[q]; done[q], when
// given, is recorded on queues[q] after its stripe.
template <typename T>
cudaError_t gemm_multi_queue(const GemmProblem<T>& p, unsigned nq, cudaStream_t* queues, cudaEvent_t* done);

// Stream-ordered workspace from the library's own per-device pool (workspace.cu).
cudaError_t ws_alloc(void** ptr, size_t bytes, cudaStream_t s);
cudaError_t ws_free(void* ptr, cudaStream_t s);
void ws_release_all();
// Number of ws_alloc calls made by the process so far (every workspace a level-3 routine takes goes
// through ws_alloc, so a call during which this does not move allocated nothing).
unsigned long long ws_alloc_count();

// One-time, per-device set-up step (a kernel's opt-in to large dynamic shared memory) that several host
// threads may reach at once: the step is idempotent, the flag is atomic.
struct DeviceOnce {
    std::atomic<unsigned char> done[64];
    template <typename F>
    cudaError_t run(F&& step)
    {
        int dev = 0;
        cudaGetDevice(&dev);
        const bool tracked = dev >= 0 && dev < 64;
        if (tracked && done[dev].load(std::memory_order_acquire)) return cudaSuccess;
        const cudaError_t e = step();
        if (e != cudaSuccess) return e;
        if (tracked) done[dev].store(1, std::memory_order_release);
        return cudaSuccess;
    }
};

// DTRSM on the fixed device-resident scratch array (no allocation); cudaErrorMemoryAllocation
// when the problem exceeds the array.
cudaError_t dtrsm_colmajor_noalloc(bool right, bool lower, bool trans, bool unit, size_t M, size_t N, double alpha,
                                   const double* A, size_t lda, double* B, size_t ldb, cudaStream_t s);

// First-use work of every FP64 GEMM kernel a triangular solve can reach without allocating, done ahead of
// time on the current device: shared-memory opt-ins and module loads.
cudaError_t dgemm_prepare_all_kernels();
cudaError_t gemm_simt_load_double_kernels();

// Fused solve of up to dtrsm_diag_fused_max_blocks() consecutive diagonal blocks of a Left-side DTRSM with few
// right-hand sides (dtrsm_diag_fused.cu).
int dtrsm_diag_fused_max_blocks();
bool dtrsm_diag_fused_applicable(const double* A, size_t lda, const double* B, size_t ldb, size_t n, size_t N);
cudaError_t launch_dtrsm_diag_fused(bool trans, bool forward, const double* A, size_t lda, size_t n, const double* inv, size_t nblk,
                                    double* B, size_t ldb, size_t N, double alpha, size_t b0, size_t b1, cudaStream_t s);
cudaError_t dtrsm_diag_fused_prepare_all();
unsigned dtrsm_fused_fault_flag();

// Sticky per-translation-unit flags set when a bounded mbarrier wait inside a kernel ran out.
unsigned dgemm_tma_fault_flag();
unsigned sgemm_tma_fault_flag();

// cuTensorMapEncodeTiled obtained through the runtime's driver entry point query (no libcuda link).
void* get_tensor_map_encoder();

// Number of SMs of the current device (cached per device).
int sm_count();

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace cb200
