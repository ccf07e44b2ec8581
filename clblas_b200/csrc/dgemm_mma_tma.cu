// DGEMM on the FP64 tensor-core path, TMA-staged: C = alpha*op(A)*op(B) + beta*C, column-major,
// for operands whose base addresses and leading dimensions are multiples of 16 bytes.
//
// This is the B200 counterpart of the reference's AutoGemm dgemm tile kernels (generator
// src/library/blas/AutoGemm/KernelOpenCL.py:13-459; hand-tuned 48x48 kernel
// src/library/blas/AutoGemm/UserGemmKernelSources/dgemm_Col_TN_B1_MX048_NX048_KX08_src.cpp).
//
// CTA = 128 x BN tile of C (BN = 128; 64 or 32 for problems too narrow to fill the SMs with 128-wide
// tiles, e.g. the panel products of TRSM), K in slabs of 16.  Warp 8 is the producer: one lane issues two TMA
// bulk-tensor loads per slab (A and B) into a STAGES-deep ring in shared memory; full/empty
// mbarriers carry the hand-over, all waits are bounded.  Warps 0-7 are consumers (2 x 4 grid,
// 64 x BN/4 of C each, up to 128 accumulator registers per thread) issuing mma.sync.m8n8k4.f64.
// TMA zero-fills whatever lies beyond M, N or K, so ragged shapes need no separate edge launches
// (the reference runs tile + row + column + corner kernels, src/library/blas/xgemm.cc:603-658);
// only the epilogue is predicated.
//
// Shared-memory layouts (both conflict-free for the m8n8k4 fragment pattern, 4 k x 8 rows):
//  * operand whose K index is contiguous in memory (A for transA=T, B for transB=N): box
//    16 (k) x 128 rows, 128-byte rows, SWIZZLE_128B.  Within every group of 8 rows the fragment row
//    g reads tile row 2*(g%4) + g/4, which spreads a half-warp over all 32 banks; the epilogue
//    applies the same permutation to the C coordinates.
//  * operand whose M/N index is contiguous (A for transA=N, B for transB=T): box (tile + 4) x 16 (k),
//    i.e. rows of 132 (68, 36) doubles of which 128 (64, 32) are used: the 4 extra elements make the
//    row pitch = 32 (mod 128) bytes, which is what separates the four k rows of a fragment.
#include "common.h"
#include "tma_pipeline.cuh"

namespace cb200 {

namespace {

constexpr int BM = 128, BK = 16;
constexpr int STAGES = 5;
constexpr int MC_PITCH = BM + 4;                    // doubles per k row of A, M-contiguous layout
constexpr int A_BYTES = 17 * 1024;                  // >= max(128*16*8, 16*132*8), multiple of 1024
constexpr int CONSUMER_WARPS = 8;
constexpr int THREADS = (CONSUMER_WARPS + 1) * 32;
constexpr int GROUP_M = 16;                         // tile rows per rasterisation group

// B operand buffer: max(BN rows of 128 bytes, 16 rows of (BN+4)*8 bytes), rounded up to 1 KB
constexpr int b_bytes(int bn) { return ((16 * (bn + 4) * 8 + 1023) / 1024) * 1024; }
constexpr int stage_bytes(int bn) { return A_BYTES + b_bytes(bn); }
constexpr int smem_bytes(int bn) { return STAGES * stage_bytes(bn) + 1024 /*alignment slack*/ + 256 /*barriers*/; }

__device__ __forceinline__ void dmma(double& c0, double& c1, double a, double b)
{
    asm volatile("mma.sync.aligned.m8n8k4.row.col.f64.f64.f64.f64 {%0,%1}, {%2}, {%3}, {%0,%1};"
                 : "+d"(c0), "+d"(c1) : "d"(a), "d"(b));
}

__device__ __forceinline__ int perm8(int g) { return 2 * (g & 3) + (g >> 2); }

// TA: A is stored K x M (K contiguous).  TB: B is stored N x K (N contiguous).
// TRI: compiled-in support for the triangular update (SYRK); without it `tri` is ignored and the epilogue carries
// no per-entry mask (a run-time mask alone cost 4-13 % on short-K products).
template <bool TA, bool TB, int BN, bool TRI>
__global__ void __launch_bounds__(THREADS, 1)
dgemm_mma_tma_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB,
                     double* __restrict__ C, size_t ldc, size_t M, size_t N, size_t K, double alpha, double beta,
                     unsigned tilesM, unsigned tilesN, unsigned wave, int tri_arg)
{
    int tri = TRI ? tri_arg : TRI_FULL;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    constexpr int STAGE_BYTES = stage_bytes(BN);
    constexpr int PITCH_B = BN + 4;                 // doubles per k row of B, N-contiguous layout
    constexpr int WN = BN / 4, NI = WN / 8;         // warp tile width, 8-wide sub-tiles per warp
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
    uint64_t* empty = full + STAGES;

    // grouped rasterisation: consecutive CTAs share A row-panels and B column-panels in L2
    unsigned tm, tn;
    {
        const unsigned per_group = GROUP_M * tilesN;
        const unsigned g = blockIdx.x / per_group;
        const unsigned first = g * GROUP_M;
        const unsigned rows = min((unsigned)GROUP_M, tilesM - first);
        const unsigned r = blockIdx.x - g * per_group;
        tm = first + r % rows;
        tn = r / rows;
    }
    const size_t m0 = (size_t)tm * BM, n0 = (size_t)tn * BN;
    if (TRI) {
        if (tri_tile_outside(tri, m0, BM, n0, BN)) return;      // triangular update: nothing of this tile is referenced
        if (tri_tile_inside(tri, m0, BM, n0, BN)) tri = TRI_FULL;
    }
    const int nk = (int)((K + BK - 1) / BK);
    // Every other wave of CTAs walks K backwards: it starts on the K range the wave before it
    // finished on, which is what L2 still holds, instead of re-streaming those panels from DRAM.
    const bool reverse_k = wave != 0 && ((blockIdx.x / wave) & 1);
    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], CONSUMER_WARPS);
        }
        mbar_fence_init();
    }
    __syncthreads();

    if (warp == CONSUMER_WARPS) {
        // ------------------------------- producer -------------------------------
        if (lane == 0) {
            tma_prefetch_descriptor(&mapA);
            tma_prefetch_descriptor(&mapB);
            for (int kt = 0; kt < nk; kt++) {
                const int s = kt % STAGES;
                if (kt >= STAGES && !mbar_wait(&empty[s], ((kt / STAGES) - 1) & 1)) break;
                unsigned char* sa = smem + s * STAGE_BYTES;
                unsigned char* sb = sa + A_BYTES;
                const uint32_t bytes = (TA ? BK * BM : MC_PITCH * BK) * 8 + (TB ? PITCH_B * BK : BK * BN) * 8;
                mbar_expect_tx(&full[s], bytes);
                const int k0 = (reverse_k ? nk - 1 - kt : kt) * BK;
                if (TA) tma_load_2d(sa, &mapA, k0, (int)m0, &full[s]); else tma_load_2d(sa, &mapA, (int)m0, k0, &full[s]);
                if (TB) tma_load_2d(sb, &mapB, (int)n0, k0, &full[s]); else tma_load_2d(sb, &mapB, k0, (int)n0, &full[s]);
            }
        }
        return;
    }

    // --------------------------------- consumers ---------------------------------
    const int wm = warp % 2, wn = warp / 2;          // 2 x 4 warps, 64 x WN each
    const int g = lane / 4, kk = lane % 4;
    const int pg = perm8(g);

    // byte offsets of this lane's fragment element inside an operand buffer, for k-step 0 and
    // sub-tile 0; sub-tiles and k-steps add compile-time constants (and one XOR for the swizzle).
    int offA, offB;
    if (TA) offA = (wm * 64 + pg) * 128 + ((((kk >> 1) ^ (pg & 1))) << 4) + (kk & 1) * 8;
    else    offA = kk * (MC_PITCH * 8) + (wm * 64 + g) * 8;
    if (!TB) offB = (wn * WN + pg) * 128 + ((((kk >> 1) ^ (pg & 1))) << 4) + (kk & 1) * 8;
    else     offB = kk * (PITCH_B * 8) + (wn * WN + g) * 8;
    const int xr = (pg & 6) << 4;                    // swizzle XOR applied to the 32-byte chunk of a k-step

    double acc[8][NI][2];
#pragma unroll
    for (int i = 0; i < 8; i++)
#pragma unroll
        for (int j = 0; j < NI; j++) acc[i][j][0] = acc[i][j][1] = 0.0;

    for (int kt = 0; kt < nk; kt++) {
        const int s = kt % STAGES;
        if (!mbar_wait(&full[s], (kt / STAGES) & 1)) break;
        const unsigned char* sa = smem + s * STAGE_BYTES;
        const unsigned char* sb = sa + A_BYTES;
#pragma unroll
        for (int ks = 0; ks < BK / 4; ks++) {
            double a[8], b[NI];
#pragma unroll
            for (int mi = 0; mi < 8; mi++) {
                const int o = TA ? offA + mi * 1024 + (((ks * 32) ^ xr))
                                 : offA + ks * 4 * (MC_PITCH * 8) + mi * 64;
                a[mi] = *reinterpret_cast<const double*>(sa + o);
            }
#pragma unroll
            for (int ni = 0; ni < NI; ni++) {
                const int o = !TB ? offB + ni * 1024 + (((ks * 32) ^ xr))
                                  : offB + ks * 4 * (PITCH_B * 8) + ni * 64;
                b[ni] = *reinterpret_cast<const double*>(sb + o);
            }
#pragma unroll
            for (int mi = 0; mi < 8; mi++)
#pragma unroll
                for (int ni = 0; ni < NI; ni++) dmma(acc[mi][ni][0], acc[mi][ni][1], a[mi], b[ni]);
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[s]);
    }

    // ---- epilogue: C = alpha*acc + beta*C; beta == 0 never reads C
    const bool useC = (beta != 0.0);
#pragma unroll
    for (int ni = 0; ni < NI; ni++)
#pragma unroll
        for (int e = 0; e < 2; e++) {
            const int j = 2 * kk + e;
            const size_t col = n0 + wn * WN + ni * 8 + (!TB ? perm8(j) : j);
            if (col >= N) continue;
            double* cc = C + col * ldc;
#pragma unroll
            for (int mi = 0; mi < 8; mi++) {
                const size_t row = m0 + wm * 64 + mi * 8 + (TA ? pg : g);
                if (row >= M || (TRI && tri_masked(tri, row, col))) continue;
                double r = alpha * acc[mi][ni][e];
                if (useC) r = fma(beta, cc[row], r);
                cc[row] = r;
            }
        }
}

template <bool TA, bool TB, int BN, bool TRI>
cudaError_t launch(const GemmProblem<double>& p, cudaStream_t s)
{
    void* enc = get_tensor_map_encoder();
    CUtensorMap mapA, mapB;
    bool ok;
    if (TA) ok = make_tensor_map_2d(&mapA, enc, CU_TENSOR_MAP_DATA_TYPE_FLOAT64, 8, p.A, p.K, p.M, p.lda, BK, BM, CU_TENSOR_MAP_SWIZZLE_128B);
    else    ok = make_tensor_map_2d(&mapA, enc, CU_TENSOR_MAP_DATA_TYPE_FLOAT64, 8, p.A, p.M, p.K, p.lda, MC_PITCH, BK, CU_TENSOR_MAP_SWIZZLE_NONE);
    if (!ok) return cudaErrorNotSupported;
    if (TB) ok = make_tensor_map_2d(&mapB, enc, CU_TENSOR_MAP_DATA_TYPE_FLOAT64, 8, p.B, p.N, p.K, p.ldb, BN + 4, BK, CU_TENSOR_MAP_SWIZZLE_NONE);
    else    ok = make_tensor_map_2d(&mapB, enc, CU_TENSOR_MAP_DATA_TYPE_FLOAT64, 8, p.B, p.K, p.N, p.ldb, BK, BN, CU_TENSOR_MAP_SWIZZLE_128B);
    if (!ok) return cudaErrorNotSupported;

    static bool attr_done[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64 || !attr_done[dev]) {
        cudaError_t e = cudaFuncSetAttribute(dgemm_mma_tma_kernel<TA, TB, BN, TRI>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes(BN));
        if (e != cudaSuccess) return e;
        if (dev >= 0 && dev < 64) attr_done[dev] = true;
    }
    const size_t tilesM = (p.M + BM - 1) / BM, tilesN = (p.N + BN - 1) / BN;
    dgemm_mma_tma_kernel<TA, TB, BN, TRI><<<(unsigned)(tilesM * tilesN), THREADS, smem_bytes(BN), s>>>(
        mapA, mapB, p.C, p.ldc, p.M, p.N, p.K, p.alpha, p.beta, (unsigned)tilesM, (unsigned)tilesN, (unsigned)(sm_count() * 1), p.tri);
    count_launch();
    return cudaGetLastError();
}

template <int BN>
cudaError_t launch_t(const GemmProblem<double>& p, cudaStream_t s)
{
    if (p.tri != TRI_FULL) {
        if (!p.ta && !p.tb) return launch<false, false, BN, true>(p, s);
        if (!p.ta && p.tb) return launch<false, true, BN, true>(p, s);
        if (p.ta && !p.tb) return launch<true, false, BN, true>(p, s);
        return launch<true, true, BN, true>(p, s);
    }
    if (!p.ta && !p.tb) return launch<false, false, BN, false>(p, s);
    if (!p.ta && p.tb) return launch<false, true, BN, false>(p, s);
    if (p.ta && !p.tb) return launch<true, false, BN, false>(p, s);
    return launch<true, true, BN, false>(p, s);
}

}  // namespace

cudaError_t launch_dgemm_mma_tma(const GemmProblem<double>& p, cudaStream_t s, int min_bn)
{
    // TMA needs 16-byte aligned global addresses and strides; coordinates are 32-bit.
    if (!aligned16(p.A) || !aligned16(p.B) || (p.lda & 1) || (p.ldb & 1)) return cudaErrorNotSupported;
    if (p.M >= (1u << 31) || p.N >= (1u << 31) || p.K >= (1u << 31)) return cudaErrorNotSupported;
    const size_t tilesM = (p.M + BM - 1) / BM;
    if (tilesM * ((p.N + 31) / 32) >= (1u << 31)) return cudaErrorNotSupported;
    set_last_kernel("dgemm_mma_tma");
    // Widest tile that still gives the 148 SMs about one CTA each; narrower tiles only for
    // problems that 128-wide tiles would leave most SMs idle on.
    if (min_bn >= 128 || tilesM * ((p.N + 127) / 128) >= 120) return launch_t<128>(p, s);
    if (tilesM * ((p.N + 63) / 64) >= 120) return launch_t<64>(p, s);
    return launch_t<32>(p, s);
}

unsigned dgemm_tma_fault_flag() { return read_wait_timeout_flag(); }

}  // namespace cb200
