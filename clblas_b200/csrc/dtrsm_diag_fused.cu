// Fused solve of up to four consecutive 128 x 128 diagonal blocks of a Left-side DTRSM for a strip of 16
// right-hand-side columns, in one launch.
//
// The blocked solve (trsm.cu; reference: the rank-128 loop of src/library/blas/xtrsm.cc:1229-1257) ends its
// recursion in chains of small dependent products: X_i = inv(A_ii) B_i, B_j -= A_ji X_i, ...  With few
// right-hand sides each of those is a launch of about a hundred small CTAs whose fixed costs (launch, pipeline
// fill, epilogue) exceed its arithmetic; for 8192 x 2048 the 96 products on 128-row blocks took 15 % of the
// solve (127 launches; 35 with this kernel).  Here one CTA carries a 16-column strip through the whole 512-row
// diagonal block:
//
//     for each 128-row block i, in substitution order:
//         acc  = sum over the blocks j already solved of op(A)[i, j] * X_j          (FP64 tensor-core MMA)
//         B_i' = alpha * B_i - acc                                                   (in shared memory)
//         X_i  = op(inv(A_ii)) * B_i'                                                (MMA), stored to B and kept
//
// The strip of B (4 x 128 x 16 doubles, 64 KB) is loaded once by TMA and stays in shared memory in the layout
// the MMA's B operand is read in (K-contiguous rows of 128 bytes, SWIZZLE_128B), so every X_i is the next
// products' operand without leaving the SM.  The A-side operands -- the off-diagonal blocks of A and the inverted
// diagonal blocks -- stream through a TMA ring exactly as in the DGEMM kernel (dgemm_mma_tma.cu), issued by a
// producer warp in the order the consumers use them.  Ten block products instead of seven launches per 512 rows;
// B is read once and written once.  All waits are bounded mbarrier waits.
#include "common.h"
#include "tma_pipeline.cuh"

#include <algorithm>
#include <cstdlib>

namespace cb200 {

namespace {

constexpr int NB = 128;                 // order of a diagonal block
constexpr int BK = 16;                  // K slab
constexpr int BN = 16;                  // right-hand-side columns per CTA
constexpr int MAX_BLOCKS = 4;           // diagonal blocks per launch
constexpr int STAGES = 4;
constexpr int MC_PITCH = NB + 4;        // doubles per k row of an M-contiguous A slab (see dgemm_mma_tma.cu)
constexpr int A_BYTES = 17 * 1024;
constexpr int X_SLAB_BYTES = BK * BN * 8;            // 2 KB: 16 n-rows of 128 bytes
constexpr int X_BLOCK_BYTES = (NB / BK) * X_SLAB_BYTES;   // 16 KB
constexpr int CONSUMER_WARPS = 8;
constexpr int THREADS = (CONSUMER_WARPS + 1) * 32;
constexpr int SMEM_BYTES = MAX_BLOCKS * X_BLOCK_BYTES + STAGES * A_BYTES + 1024 + 256;

__device__ __forceinline__ void dmma(double& c0, double& c1, double a, double b)
{
    asm volatile("mma.sync.aligned.m8n8k4.row.col.f64.f64.f64.f64 {%0,%1}, {%2}, {%3}, {%0,%1};"
                 : "+d"(c0), "+d"(c1) : "d"(a), "d"(b));
}
__device__ __forceinline__ int perm8(int g) { return 2 * (g & 3) + (g >> 2); }
__device__ __forceinline__ void consumer_barrier() { asm volatile("bar.sync 1, 256;" ::: "memory"); }

// TA: op(A) = A^T, i.e. the blocks of A and of the inverses are read K-contiguous.
// blk0: first diagonal block of the range, nb its length, forward: substitution runs from blk0 upwards.
template <bool TA>
__global__ void __launch_bounds__(THREADS, 1)
dtrsm_diag_fused_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapInv,
                        const __grid_constant__ CUtensorMap mapB, double* __restrict__ B, size_t ldb, size_t n, size_t N,
                        double alpha, unsigned blk0, unsigned nb, int forward)
{
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    unsigned char* xbuf = smem;                                         // nb x 16 KB, B-operand layout
    unsigned char* ring = smem + MAX_BLOCKS * X_BLOCK_BYTES;
    uint64_t* full = reinterpret_cast<uint64_t*>(ring + STAGES * A_BYTES);
    uint64_t* empty = full + STAGES;
    uint64_t* rhs_full = empty + STAGES;

    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const size_t n0 = (size_t)blockIdx.x * BN;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], CONSUMER_WARPS);
        }
        mbar_init(rhs_full, 1);
        mbar_fence_init();
    }
    __syncthreads();
    pdl_wait();

    // block handled at step t of the substitution
    auto block_at = [&](unsigned t) { return forward ? blk0 + t : blk0 + nb - 1 - t; };

    if (warp == CONSUMER_WARPS) {
        // ------------------------------- producer -------------------------------
        if (lane == 0) {
            tma_prefetch_descriptor(&mapA);
            tma_prefetch_descriptor(&mapInv);
            tma_prefetch_descriptor(&mapB);
            // the strip of B: block t of the range lands in xbuf slot t (slot order = memory order of the range)
            mbar_expect_tx(rhs_full, nb * X_BLOCK_BYTES);
            for (unsigned q = 0; q < nb; q++)
                for (int s = 0; s < NB / BK; s++)
                    tma_load_2d(xbuf + q * X_BLOCK_BYTES + s * X_SLAB_BYTES, &mapB, (int)((blk0 + q) * NB + s * BK), (int)n0, rhs_full);
            unsigned it = 0;
            for (unsigned t = 0; t < nb; t++) {
                const unsigned bi = block_at(t);
                for (unsigned u = 0; u <= t; u++) {
                    // u < t: off-diagonal block op(A)[bi, bj] with bj solved at step u; u == t: the inverse of block bi
                    const bool diag = (u == t);
                    const unsigned bj = block_at(u);
                    for (int s = 0; s < NB / BK; s++, it++) {
                        const int st = (int)(it % STAGES);
                        if (it >= STAGES && !mbar_wait(&empty[st], ((it / STAGES) - 1) & 1)) return;
                        unsigned char* sa = ring + st * A_BYTES;
                        mbar_expect_tx(&full[st], (TA ? BK * NB : MC_PITCH * BK) * 8);
                        if (diag) {
                            // inverses: block b is columns [128 b, 128 b + 128) of a 128-row matrix
                            if (TA) tma_load_2d(sa, &mapInv, s * BK, (int)(bi * NB), &full[st]);
                            else    tma_load_2d(sa, &mapInv, 0, (int)(bi * NB + s * BK), &full[st]);
                        } else {
                            if (TA) tma_load_2d(sa, &mapA, (int)(bj * NB + s * BK), (int)(bi * NB), &full[st]);
                            else    tma_load_2d(sa, &mapA, (int)(bi * NB), (int)(bj * NB + s * BK), &full[st]);
                        }
                    }
                }
            }
        }
        return;
    }

    // --------------------------------- consumers ---------------------------------
    // warp w owns rows [16 w, 16 w + 16) of every block and all 16 columns: 2 x 2 MMA sub-tiles
    const int g = lane / 4, kk = lane % 4;
    const int pg = perm8(g);
    int offA;
    if (TA) offA = (warp * 16 + pg) * 128 + ((((kk >> 1) ^ (pg & 1))) << 4) + (kk & 1) * 8;
    else    offA = kk * (MC_PITCH * 8) + (warp * 16 + g) * 8;
    const int offB = pg * 128 + ((((kk >> 1) ^ (pg & 1))) << 4) + (kk & 1) * 8;
    const int xr = (pg & 6) << 4;

    double acc[2][2][2];
    auto clear = [&]() {
#pragma unroll
        for (int mi = 0; mi < 2; mi++)
#pragma unroll
            for (int ni = 0; ni < 2; ni++) acc[mi][ni][0] = acc[mi][ni][1] = 0.0;
    };
    unsigned it = 0;
    // acc += (the next 8 slabs of the ring) * (the block in xbuf slot q)
    auto block_product = [&](unsigned q) -> bool {
        const unsigned char* xb = xbuf + q * X_BLOCK_BYTES;
        for (int s = 0; s < NB / BK; s++, it++) {
            const int st = (int)(it % STAGES);
            if (!mbar_wait(&full[st], (it / STAGES) & 1)) return false;
            const unsigned char* sa = ring + st * A_BYTES;
            const unsigned char* sb = xb + s * X_SLAB_BYTES;
#pragma unroll
            for (int ks = 0; ks < BK / 4; ks++) {
                double a[2], b[2];
#pragma unroll
                for (int mi = 0; mi < 2; mi++) {
                    const int o = TA ? offA + mi * 1024 + ((ks * 32) ^ xr) : offA + ks * 4 * (MC_PITCH * 8) + mi * 64;
                    a[mi] = *reinterpret_cast<const double*>(sa + o);
                }
#pragma unroll
                for (int ni = 0; ni < 2; ni++) b[ni] = *reinterpret_cast<const double*>(sb + offB + ni * 1024 + ((ks * 32) ^ xr));
#pragma unroll
                for (int mi = 0; mi < 2; mi++)
#pragma unroll
                    for (int ni = 0; ni < 2; ni++) dmma(acc[mi][ni][0], acc[mi][ni][1], a[mi], b[ni]);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[st]);
        }
        return true;
    };
    // where this lane's accumulator element (mi, ni, e) lives: row inside the block, column inside the strip, and
    // its address in a block of xbuf (as a B operand the element is k = row, n = column)
    auto elem_row = [&](int mi) { return warp * 16 + mi * 8 + (TA ? pg : g); };
    auto elem_col = [&](int ni, int e) { return ni * 8 + perm8(2 * kk + e); };
    auto elem_ptr = [&](unsigned q, int mi, int ni, int e) {
        const int row = elem_row(mi), col = elem_col(ni, e), k = row % BK;
        return reinterpret_cast<double*>(xbuf + q * X_BLOCK_BYTES + (row / BK) * X_SLAB_BYTES + col * 128 +
                                         ((((k >> 1) ^ (col & 7)) << 4) | ((k & 1) << 3)));
    };

    if (!mbar_wait(rhs_full, 0)) return;
    for (unsigned t = 0; t < nb; t++) {
        const unsigned bi = block_at(t);
        const unsigned qi = bi - blk0;                      // xbuf slot of block bi
        clear();
        for (unsigned u = 0; u < t; u++)
            if (!block_product(block_at(u) - blk0)) return;
        // B_i' = alpha * B_i - acc, every lane on its own elements
#pragma unroll
        for (int mi = 0; mi < 2; mi++)
#pragma unroll
            for (int ni = 0; ni < 2; ni++)
#pragma unroll
                for (int e = 0; e < 2; e++) {
                    double* p = elem_ptr(qi, mi, ni, e);
                    *p = alpha * *p - acc[mi][ni][e];
                }
        consumer_barrier();                                 // B_i' complete before it is an operand
        clear();
        if (!block_product(qi)) return;
        consumer_barrier();                                 // every warp has read B_i' before X_i replaces it
#pragma unroll
        for (int mi = 0; mi < 2; mi++)
#pragma unroll
            for (int ni = 0; ni < 2; ni++)
#pragma unroll
                for (int e = 0; e < 2; e++) {
                    *elem_ptr(qi, mi, ni, e) = acc[mi][ni][e];
                    const size_t row = (size_t)bi * NB + elem_row(mi), col = n0 + elem_col(ni, e);
                    if (row < n && col < N) B[row + col * ldb] = acc[mi][ni][e];
                }
        if (t + 1 < nb) consumer_barrier();                 // X_i visible to the products of the next block
    }
}

DeviceOnce g_once[2];

template <bool TA>
cudaError_t prepare()
{
    return g_once[TA].run([] {
        return cudaFuncSetAttribute(dtrsm_diag_fused_kernel<TA>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    });
}

}  // namespace

int dtrsm_diag_fused_max_blocks() { return MAX_BLOCKS; }

bool dtrsm_diag_fused_applicable(const double* A, size_t lda, const double* B, size_t ldb, size_t n, size_t N)
{
    // Measured with and without (TFLOP/s): 8192 x 2048 30.1 / 27.3, 8192 x 4096 31.3 / 29.5, 8192 x 16384 32.9 / 32.0,
    // 4096 x 1024 19.3 / 16.2 -- it pays at every width, so there is no upper limit on N.
    if (N == 0) return false;
    if (!aligned16(A) || !aligned16(B) || (lda & 1) || (ldb & 1)) return false;
    if (n >= (1u << 31) || N >= (1u << 31)) return false;
    return get_tensor_map_encoder() != nullptr;
}

// Solves the diagonal blocks [b0, b1) (b1 - b0 <= 4) of op(A) X = alpha B for all N columns; inv holds the
// inverted 128 x 128 diagonal blocks.  forward: op(A) is lower triangular (block b0 first).
cudaError_t launch_dtrsm_diag_fused(bool trans, bool forward, const double* A, size_t lda, size_t n, const double* inv, size_t nblk,
                                    double* B, size_t ldb, size_t N, double alpha, size_t b0, size_t b1, cudaStream_t s)
{
    if (b1 <= b0 || b1 - b0 > (size_t)MAX_BLOCKS) return cudaErrorInvalidValue;
    void* enc = get_tensor_map_encoder();
    CUtensorMap mapA, mapInv, mapB;
    bool ok;
    if (trans) {
        ok = make_tensor_map_2d(&mapA, enc, CU_TENSOR_MAP_DATA_TYPE_FLOAT64, 8, A, n, n, lda, BK, NB, CU_TENSOR_MAP_SWIZZLE_128B) &&
             make_tensor_map_2d(&mapInv, enc, CU_TENSOR_MAP_DATA_TYPE_FLOAT64, 8, inv, NB, nblk * NB, NB, BK, NB, CU_TENSOR_MAP_SWIZZLE_128B);
    } else {
        ok = make_tensor_map_2d(&mapA, enc, CU_TENSOR_MAP_DATA_TYPE_FLOAT64, 8, A, n, n, lda, MC_PITCH, BK, CU_TENSOR_MAP_SWIZZLE_NONE) &&
             make_tensor_map_2d(&mapInv, enc, CU_TENSOR_MAP_DATA_TYPE_FLOAT64, 8, inv, NB, nblk * NB, NB, MC_PITCH, BK, CU_TENSOR_MAP_SWIZZLE_NONE);
    }
    ok = ok && make_tensor_map_2d(&mapB, enc, CU_TENSOR_MAP_DATA_TYPE_FLOAT64, 8, B, n, N, ldb, BK, BN, CU_TENSOR_MAP_SWIZZLE_128B);
    if (!ok) return cudaErrorNotSupported;
    cudaError_t e = trans ? prepare<true>() : prepare<false>();
    if (e != cudaSuccess) return e;
    const dim3 grid((unsigned)((N + BN - 1) / BN)), block(THREADS);
    if (trans) e = launch_pdl(dtrsm_diag_fused_kernel<true>, grid, block, SMEM_BYTES, s, mapA, mapInv, mapB, B, ldb, n, N, alpha,
                              (unsigned)b0, (unsigned)(b1 - b0), forward ? 1 : 0);
    else       e = launch_pdl(dtrsm_diag_fused_kernel<false>, grid, block, SMEM_BYTES, s, mapA, mapInv, mapB, B, ldb, n, N, alpha,
                              (unsigned)b0, (unsigned)(b1 - b0), forward ? 1 : 0);
    count_launch();
    return e;
}

cudaError_t dtrsm_diag_fused_prepare_all()
{
    cudaFuncAttributes fa;
    cudaError_t e;
    if ((e = prepare<false>()) != cudaSuccess) return e;
    if ((e = cudaFuncGetAttributes(&fa, dtrsm_diag_fused_kernel<false>)) != cudaSuccess) return e;
    if ((e = prepare<true>()) != cudaSuccess) return e;
    return cudaFuncGetAttributes(&fa, dtrsm_diag_fused_kernel<true>);
}

unsigned dtrsm_fused_fault_flag() { return read_wait_timeout_flag(); }

}  // namespace cb200
