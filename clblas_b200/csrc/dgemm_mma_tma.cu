// DGEMM on the FP64 tensor-core path, TMA-staged: C = alpha*op(A)*op(B) + beta*C, column-major,
// for operands whose base addresses and leading dimensions are multiples of 16 bytes.
//
// This is the B200 counterpart of the reference's AutoGemm dgemm tile kernels (generator
// src/library/blas/AutoGemm/KernelOpenCL.py:13-459; hand-tuned 48x48 kernel
// src/library/blas/AutoGemm/UserGemmKernelSources/dgemm_Col_TN_B1_MX048_NX048_KX08_src.cpp).
//
// CTA = 128 x BN tile of C (BN = 128; 64, 32 or 16 for problems too narrow to fill the SMs with 128-wide
// tiles, e.g. the panel products of TRSM), K in slabs of 16.  Warp 8 is the producer: one lane issues two TMA
// bulk-tensor loads per slab (A and B) into a STAGES-deep ring in shared memory; full/empty
// mbarriers carry the hand-over, all waits are bounded.  Warps 0-7 are consumers (2 x 4 grid,
// 64 x BN/4 of C each, up to 128 accumulator registers per thread; 8 x 1 grid, 16 x 16 each, for BN = 16)
// issuing mma.sync.m8n8k4.f64.
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

#include <algorithm>
#include <cstdio>
#include <cstdlib>
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
    constexpr int WARPS_M = BN >= 32 ? 2 : 8;       // consumer warps along M and along N
    constexpr int WARPS_N = CONSUMER_WARPS / WARPS_M;
    constexpr int WM = BM / WARPS_M, MI = WM / 8;   // warp tile height, 8-high sub-tiles per warp
    constexpr int WN = BN / WARPS_N, NI = WN / 8;   // warp tile width, 8-wide sub-tiles per warp
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
    uint64_t* empty = full + STAGES;
    pdl_launch_dependents();

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
    pdl_wait();               // everything below reads or writes global memory

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
    const int wm = warp % WARPS_M, wn = warp / WARPS_M;          // WARPS_M x WARPS_N warps, WM x WN each
    const int g = lane / 4, kk = lane % 4;
    const int pg = perm8(g);

    // byte offsets of this lane's fragment element inside an operand buffer, for k-step 0 and
    // sub-tile 0; sub-tiles and k-steps add compile-time constants (and one XOR for the swizzle).
    int offA, offB;
    if (TA) offA = (wm * WM + pg) * 128 + ((((kk >> 1) ^ (pg & 1))) << 4) + (kk & 1) * 8;
    else    offA = kk * (MC_PITCH * 8) + (wm * WM + g) * 8;
    if (!TB) offB = (wn * WN + pg) * 128 + ((((kk >> 1) ^ (pg & 1))) << 4) + (kk & 1) * 8;
    else     offB = kk * (PITCH_B * 8) + (wn * WN + g) * 8;
    const int xr = (pg & 6) << 4;                    // swizzle XOR applied to the 32-byte chunk of a k-step

    double acc[MI][NI][2];
#pragma unroll
    for (int i = 0; i < MI; i++)
#pragma unroll
        for (int j = 0; j < NI; j++) acc[i][j][0] = acc[i][j][1] = 0.0;

    for (int kt = 0; kt < nk; kt++) {
        const int s = kt % STAGES;
        if (!mbar_wait(&full[s], (kt / STAGES) & 1)) break;
        const unsigned char* sa = smem + s * STAGE_BYTES;
        const unsigned char* sb = sa + A_BYTES;
#pragma unroll
        for (int ks = 0; ks < BK / 4; ks++) {
            double a[MI], b[NI];
#pragma unroll
            for (int mi = 0; mi < MI; mi++) {
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
            for (int mi = 0; mi < MI; mi++)
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
            for (int mi = 0; mi < MI; mi++) {
                const size_t row = m0 + wm * WM + mi * 8 + (TA ? pg : g);
                if (row >= M || (TRI && tri_masked(tri, row, col))) continue;
                double r = alpha * acc[mi][ni][e];
                if (useC) r = fma(beta, cc[row], r);
                cc[row] = r;
            }
        }
}

// ---------------------------------------------------------------------------------------------
// Tail of the grid, shared between all SMs ("stream-K" for the last partial wave).
//
// With one CTA per tile, a grid of T tiles on S SMs runs ceil(T / S) waves; the last one keeps only T mod S SMs
// busy (DGEMM 2048^3: 256 tiles = 1.73 waves, two waves of time).  The main kernel therefore takes the first
// floor(T / S) * S tiles and this kernel the R = T mod S remaining ones: their R * nk K-slabs are cut into equal
// consecutive shares, one per CTA, so a CTA computes part of one tile (sometimes the end of one and the start of
// the next).  A CTA that owns a whole tile writes C directly.  Otherwise it stores its partial tile into its slot of
// a workspace and takes a ticket from the tile's counter; the CTA that draws the last ticket adds the slots in slot
// order -- a fixed order, so the result does not depend on which CTA finishes last -- and writes C.  Nobody waits
// for anybody: there is no spin loop in this kernel besides the bounded mbarrier waits of the TMA ring.
constexpr int SK_MIN_SLABS = 8;          // smallest share of a CTA, in K slabs of 16

__device__ __forceinline__ void tile_coords(unsigned tile, unsigned tilesM, unsigned tilesN, unsigned& tm, unsigned& tn)
{
    const unsigned per_group = GROUP_M * tilesN;
    const unsigned g = tile / per_group;
    const unsigned first = g * GROUP_M;
    const unsigned rows = min((unsigned)GROUP_M, tilesM - first);
    const unsigned r = tile - g * per_group;
    tm = first + r % rows;
    tn = r / rows;
}

// TRI: a triangular update; the tiles are then those that touch the triangle, in the order of tri_tile_coords, and tiles
// on the diagonal mask their stores.
template <bool TA, bool TB, bool TRI>
__global__ void __launch_bounds__(THREADS, 1)
dgemm_streamk_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB,
                     double* __restrict__ C, size_t ldc, size_t M, size_t N, size_t K, double alpha, double beta,
                     unsigned tilesM, unsigned tilesN, unsigned tile0, unsigned units, unsigned upc,
                     double* __restrict__ ws, unsigned* __restrict__ counters, int tri)
{
    auto coords = [&](unsigned tile, unsigned& tm, unsigned& tn) {
        if (TRI) tri_tile_coords(tri, tile, tilesM, tilesN, tm, tn);
        else tile_coords(tile, tilesM, tilesN, tm, tn);
    };
    constexpr int BN = 128;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    constexpr int STAGE_BYTES = stage_bytes(BN);
    constexpr int PITCH_B = BN + 4;
    constexpr int WN = BN / 4, NI = WN / 8;
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
    uint64_t* empty = full + STAGES;
    unsigned* s_ticket = reinterpret_cast<unsigned*>(empty + STAGES);

    pdl_launch_dependents();
    const unsigned nk = (unsigned)((K + BK - 1) / BK);
    const unsigned u0 = blockIdx.x * upc, u1 = min(u0 + upc, units);
    if (u0 >= u1) return;
    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], CONSUMER_WARPS);
        }
        mbar_fence_init();
    }
    __syncthreads();
    pdl_wait();

    if (warp == CONSUMER_WARPS) {
        // ------------------------------- producer -------------------------------
        if (lane == 0) {
            tma_prefetch_descriptor(&mapA);
            tma_prefetch_descriptor(&mapB);
            unsigned t = u0 / nk, kt = u0 % nk, tm, tn;
            coords(tile0 + t, tm, tn);
            for (unsigned u = u0; u < u1; u++) {
                const unsigned i = u - u0;
                const int s = (int)(i % STAGES);
                if (i >= STAGES && !mbar_wait(&empty[s], ((i / STAGES) - 1) & 1)) break;
                unsigned char* sa = smem + s * STAGE_BYTES;
                unsigned char* sb = sa + A_BYTES;
                const uint32_t bytes = (TA ? BK * BM : MC_PITCH * BK) * 8 + (TB ? PITCH_B * BK : BK * BN) * 8;
                mbar_expect_tx(&full[s], bytes);
                const int k0 = (int)(kt * BK), m0 = (int)(tm * BM), n0 = (int)(tn * BN);
                if (TA) tma_load_2d(sa, &mapA, k0, m0, &full[s]); else tma_load_2d(sa, &mapA, m0, k0, &full[s]);
                if (TB) tma_load_2d(sb, &mapB, n0, k0, &full[s]); else tma_load_2d(sb, &mapB, k0, n0, &full[s]);
                if (++kt == nk) { kt = 0; t++; if (u + 1 < u1) coords(tile0 + t, tm, tn); }
            }
        }
        return;
    }

    // --------------------------------- consumers ---------------------------------
    const int wm = warp % 2, wn = warp / 2;
    const int g = lane / 4, kk = lane % 4;
    const int pg = perm8(g);
    const int ctid = threadIdx.x;                    // 0..255: the consumer warps are warps 0..7
    int offA, offB;
    if (TA) offA = (wm * 64 + pg) * 128 + ((((kk >> 1) ^ (pg & 1))) << 4) + (kk & 1) * 8;
    else    offA = kk * (MC_PITCH * 8) + (wm * 64 + g) * 8;
    if (!TB) offB = (wn * WN + pg) * 128 + ((((kk >> 1) ^ (pg & 1))) << 4) + (kk & 1) * 8;
    else     offB = kk * (PITCH_B * 8) + (wn * WN + g) * 8;
    const int xr = (pg & 6) << 4;

    double acc[8][NI][2];
#pragma unroll
    for (int i = 0; i < 8; i++)
#pragma unroll
        for (int j = 0; j < NI; j++) acc[i][j][0] = acc[i][j][1] = 0.0;

    // C = alpha*acc + beta*C for the tile at (m0, n0); beta == 0 never reads C
    auto epilogue = [&](size_t m0, size_t n0) {
        const bool useC = (beta != 0.0);
        const int trimode = TRI && !tri_tile_inside(tri, m0, BM, n0, BN) ? tri : TRI_FULL;
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
                    if (row >= M) continue;
                    if (TRI && tri_masked(trimode, row, col)) continue;
                    double r = alpha * acc[mi][ni][e];
                    if (useC) r = fma(beta, cc[row], r);
                    cc[row] = r;
                }
            }
    };

    // Outer loop over this CTA's segments (one per tile it touches), inner loop over the K slabs of a segment: the
    // inner loop is the main kernel's, so it keeps that kernel's register allocation.
    unsigned u = u0;
    while (u < u1) {
        const unsigned t = u / nk, seg_first = u - t * nk;
        const unsigned seg_end = min(u1, (t + 1) * nk);          // one past the last unit of this segment
        for (unsigned i = u - u0; i < seg_end - u0; i++) {
            const int s = (int)(i % STAGES);
            if (!mbar_wait(&full[s], (i / STAGES) & 1)) return;   // flagged; C of this tile stays unwritten
            const unsigned char* sa = smem + s * STAGE_BYTES;
            const unsigned char* sb = sa + A_BYTES;
#pragma unroll
            for (int ks = 0; ks < BK / 4; ks++) {
                double a[8], b[NI];
#pragma unroll
                for (int mi = 0; mi < 8; mi++) {
                    const int o = TA ? offA + mi * 1024 + (((ks * 32) ^ xr)) : offA + ks * 4 * (MC_PITCH * 8) + mi * 64;
                    a[mi] = *reinterpret_cast<const double*>(sa + o);
                }
#pragma unroll
                for (int ni = 0; ni < NI; ni++) {
                    const int o = !TB ? offB + ni * 1024 + (((ks * 32) ^ xr)) : offB + ks * 4 * (PITCH_B * 8) + ni * 64;
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

        // ---- end of this CTA's segment [seg_first, seg_last] of tile t
        const unsigned seg_last = seg_end - 1 - t * nk;
        unsigned tm, tn;
        coords(tile0 + t, tm, tn);
        const size_t m0 = (size_t)tm * BM, n0 = (size_t)tn * BN;
        if (seg_first == 0 && seg_last == nk - 1) {
            epilogue(m0, n0);
        } else {
            // Two slots per CTA: a partial tile is either the CTA's first segment (slot 0) or, begun at a tile boundary and
            // cut short by the end of the share, its last (slot 1); whole tiles in between need none.
            const unsigned first_cta = (t * nk) / upc;
            const unsigned count = ((t + 1) * nk - 1) / upc - first_cta + 1;
            double* slot = ws + ((size_t)blockIdx.x * 2 + (u == u0 ? 0 : 1)) * (size_t)(BM * BN);
#pragma unroll
            for (int mi = 0; mi < 8; mi++)
#pragma unroll
                for (int ni = 0; ni < NI; ni++)
#pragma unroll
                    for (int e = 0; e < 2; e++) __stcg(slot + ((mi * NI + ni) * 2 + e) * 256 + ctid, acc[mi][ni][e]);
            __threadfence();
            asm volatile("bar.sync 1, 256;" ::: "memory");
            if (ctid == 0) *s_ticket = atomicAdd(&counters[t], 1u);
            asm volatile("bar.sync 1, 256;" ::: "memory");
            if (*s_ticket == count - 1) {
                __threadfence();
                // slot by slot (the 64 loads of a slot are independent and overlap; a loop over the slots inside each
                // element would be a chain of dependent L2 latencies), always in slot order

#pragma unroll
                for (int mi = 0; mi < 8; mi++)
#pragma unroll
                    for (int ni = 0; ni < NI; ni++) acc[mi][ni][0] = acc[mi][ni][1] = 0.0;
                for (unsigned c = first_cta; c < first_cta + count; c++) {
                    // CTA c's part of this tile is its first segment if its share starts inside the tile
                    const double* sl = ws + ((size_t)c * 2 + (c * upc >= t * nk ? 0 : 1)) * (size_t)(BM * BN) + ctid;
                    double v[8][NI][2];
#pragma unroll
                    for (int mi = 0; mi < 8; mi++)
#pragma unroll
                        for (int ni = 0; ni < NI; ni++)
#pragma unroll
                            for (int e = 0; e < 2; e++) v[mi][ni][e] = __ldcg(sl + ((mi * NI + ni) * 2 + e) * 256);
#pragma unroll
                    for (int mi = 0; mi < 8; mi++)
#pragma unroll
                        for (int ni = 0; ni < NI; ni++)
#pragma unroll
                            for (int e = 0; e < 2; e++) acc[mi][ni][e] += v[mi][ni][e];
                }
                epilogue(m0, n0);
            }
            asm volatile("bar.sync 1, 256;" ::: "memory");      // s_ticket is reused by the next segment
        }
#pragma unroll
        for (int mi = 0; mi < 8; mi++)
#pragma unroll
            for (int ni = 0; ni < NI; ni++) acc[mi][ni][0] = acc[mi][ni][1] = 0.0;
        u = seg_end;
    }
}

// One-time per-device opt-in to the kernels' dynamic shared memory.
template <bool TA, bool TB, int BN, bool TRI>
cudaError_t prepare_main()
{
    static DeviceOnce once;
    return once.run([] {
        return cudaFuncSetAttribute(dgemm_mma_tma_kernel<TA, TB, BN, TRI>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes(BN));
    });
}
template <bool TA, bool TB, bool TRI = false>
cudaError_t prepare_streamk()
{
    static DeviceOnce once;
    return once.run([] {
        return cudaFuncSetAttribute(dgemm_streamk_kernel<TA, TB, TRI>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes(128));
    });
}

// A triangular update that the stream-K kernel should take whole: a last wave of one CTA per tile that would be less than
// 85 % full, at least 12 K slabs per SM in all, at most 16 waves of tiles in the triangle.  DSYRK Lower/N n = k, TFLOP/s,
// one CTA per tile -> stream-K: 1024 12.4 -> 15.5, 1536 16.0 -> 24.2, 2560 22.4 -> 28.9, 3072 21.9 -> 30.4, 4096 29.5 -> 32.1,
// 5120 31.2 -> 33.0, 8192 32.6 -> 34.0; not 2048 (136 tiles, one nearly full wave: 28.6 against 27.7) nor 6144 (7.95 waves:
// 33.9 against 33.5).
constexpr size_t DGEMM_TRI_SK_MAX_WAVES = 16, DGEMM_TRI_SK_MIN_SLABS_PER_SM = 12;
bool dgemm_tri_streamk_applies(const GemmProblem<double>& p)
{
    if (p.tri == TRI_FULL || !gemm_may_allocate() || p.C == p.A || p.C == p.B || getenv("CLBLAS_B200_NO_STREAMK") != nullptr) return false;
    const size_t tilesM = (p.M + BM - 1) / BM, tilesN = (p.N + 127) / 128, nk = (p.K + BK - 1) / BK, S = (size_t)sm_count();
    const size_t T = tri_tile_count(p.tri, tilesM, tilesN), R = T % S;
    if (R == 0 || R * 20 > S * 17) return false;                // the last wave of one CTA per tile is (nearly) full
    return nk >= 2 * SK_MIN_SLABS && nk < (1u << 20) && T * nk >= S * DGEMM_TRI_SK_MIN_SLABS_PER_SM && T <= S * DGEMM_TRI_SK_MAX_WAVES &&
           T * nk < (1ull << 31);
}

// "dgemm_mma_tma<T,N,128>" (+ "+tri", "+streamk_tail" / "+streamk"): the instantiation a call ran, for the tests.
const char* variant_name(bool ta, bool tb, int bn, bool tri, bool streamk)
{
    static thread_local char buf[64];
    snprintf(buf, sizeof(buf), "dgemm_mma_tma<%c,%c,%d>%s%s", ta ? 'T' : 'N', tb ? 'T' : 'N', bn, tri ? "+tri" : "",
             !streamk ? "" : tri ? "+streamk" : "+streamk_tail");
    return buf;
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

    cudaError_t e0 = prepare_main<TA, TB, BN, TRI>();
    if (e0 != cudaSuccess) return e0;
    const size_t tilesM = (p.M + BM - 1) / BM, tilesN = (p.N + BN - 1) / BN;
    size_t main_tiles = tilesM * tilesN;
    if (BN == 128 && TRI && dgemm_tri_streamk_applies(p)) {
        // Triangular update: the tiles that touch the triangle, all of them through the stream-K kernel in equal shares.  With
        // one CTA per tile they come in partly filled waves (order 3072: 300 tiles on 148 SMs, three waves for two of work).
        const size_t T = tri_tile_count(p.tri, tilesM, tilesN), S = (size_t)sm_count(), nk = (p.K + BK - 1) / BK;
        const size_t units = T * nk;
        const size_t ctas = std::max<size_t>(1, std::min<size_t>(S, units / SK_MIN_SLABS));
        const size_t upc = (units + ctas - 1) / ctas, grid = (units + upc - 1) / upc;
        const size_t ws_doubles = grid * 2 * (size_t)(BM * 128);               // two partial-tile slots per CTA
        double* ws = nullptr;
        cudaError_t e = ws_alloc(reinterpret_cast<void**>(&ws), ws_doubles * sizeof(double) + T * sizeof(unsigned) + 256, s);
        if (e == cudaSuccess) {
            unsigned* counters = reinterpret_cast<unsigned*>(ws + ws_doubles);
            e = cudaMemsetAsync(counters, 0, T * sizeof(unsigned), s);
            if (e == cudaSuccess) e = prepare_streamk<TA, TB, true>();
            if (e == cudaSuccess) {
                set_last_variant(variant_name(TA, TB, BN, true, true));
                e = launch_pdl(dgemm_streamk_kernel<TA, TB, true>, dim3((unsigned)grid), dim3(THREADS), smem_bytes(128), s,
                               mapA, mapB, p.C, p.ldc, p.M, p.N, p.K, p.alpha, p.beta, (unsigned)tilesM, (unsigned)tilesN,
                               0u, (unsigned)units, (unsigned)upc, ws, counters, p.tri);
                count_launch();
            }
            const cudaError_t e2 = ws_free(ws, s);
            return e != cudaSuccess ? e : e2;
        }
        cudaGetLastError();        // no workspace: one CTA per tile as usual
    }
    if (BN == 128 && !TRI) {
        // Whole waves go to the kernel above, the last partial wave to the stream-K kernel.  A product of fewer tiles than
        // SMs with a long K loop is one partial wave: all of it goes to the stream-K kernel, every SM working the same
        // number of slabs.  It pays from about 40 slabs per SM on (TFLOP/s, with / narrow tiles instead: 1280^3 27.5 / 20.9,
        // 1024 x 1024 x 8192 33.7 / 29.0; but 1024^3, 28 slabs per SM, 22.8 / 25.7).
        const size_t T = tilesM * tilesN, S = (size_t)sm_count(), R = T % S, nk = (p.K + BK - 1) / BK;
        const bool tail = T > S && R != 0 && R * 20 <= S * 17;
        const bool whole = T < S && T * 20 <= S * 19 && T * nk >= S * 40;
        if ((tail || whole) && nk >= 2 * SK_MIN_SLABS && nk < (1u << 20) && gemm_may_allocate() &&
            p.C != p.A && p.C != p.B && getenv("CLBLAS_B200_NO_STREAMK") == nullptr) {
            const size_t units = R * nk;
            const size_t ctas = std::max<size_t>(1, std::min<size_t>(S, units / SK_MIN_SLABS));
            const size_t upc = (units + ctas - 1) / ctas, grid = (units + upc - 1) / upc;
            const size_t ws_doubles = grid * 2 * (size_t)(BM * 128);               // two partial-tile slots per CTA
            double* ws = nullptr;
            cudaError_t e = ws_alloc(reinterpret_cast<void**>(&ws), ws_doubles * sizeof(double) + R * sizeof(unsigned) + 256, s);
            if (e == cudaSuccess) {
                unsigned* counters = reinterpret_cast<unsigned*>(ws + ws_doubles);
                e = cudaMemsetAsync(counters, 0, R * sizeof(unsigned), s);
                if (e == cudaSuccess) e = prepare_streamk<TA, TB, false>();
                if (e == cudaSuccess) {
                    main_tiles = T - R;
                    set_last_variant(variant_name(TA, TB, BN, TRI, true));
                    if (main_tiles > 0) {
                        e = launch_pdl(dgemm_mma_tma_kernel<TA, TB, BN, TRI>, dim3((unsigned)main_tiles), dim3(THREADS), smem_bytes(BN), s,
                                       mapA, mapB, p.C, p.ldc, p.M, p.N, p.K, p.alpha, p.beta, (unsigned)tilesM, (unsigned)tilesN, (unsigned)S, p.tri);
                        count_launch();
                    }
                    if (e == cudaSuccess) {
                        e = launch_pdl(dgemm_streamk_kernel<TA, TB, false>, dim3((unsigned)grid), dim3(THREADS), smem_bytes(128), s,
                                       mapA, mapB, p.C, p.ldc, p.M, p.N, p.K, p.alpha, p.beta, (unsigned)tilesM, (unsigned)tilesN,
                                       (unsigned)main_tiles, (unsigned)units, (unsigned)upc, ws, counters, 0);
                        count_launch();
                    }
                }
                const cudaError_t e2 = ws_free(ws, s);
                return e != cudaSuccess ? e : e2;
            }
            cudaGetLastError();        // no workspace: one CTA per tile as usual
        }
    }
    set_last_variant(variant_name(TA, TB, BN, TRI, false));
    const cudaError_t e = launch_pdl(dgemm_mma_tma_kernel<TA, TB, BN, TRI>, dim3((unsigned)main_tiles), dim3(THREADS), smem_bytes(BN), s,
                                     mapA, mapB, p.C, p.ldc, p.M, p.N, p.K, p.alpha, p.beta, (unsigned)tilesM, (unsigned)tilesN,
                                     (unsigned)(sm_count() * 1), p.tri);
    count_launch();
    return e;
}

// Shared-memory opt-in and module load of every instantiation without the triangular mode (what a
// triangular solve can dispatch to when it may not allocate).
template <bool TA, bool TB>
cudaError_t prepare_transposition()
{
    cudaFuncAttributes fa;
    cudaError_t e;
    if ((e = prepare_main<TA, TB, 128, false>()) != cudaSuccess) return e;
    if ((e = cudaFuncGetAttributes(&fa, dgemm_mma_tma_kernel<TA, TB, 128, false>)) != cudaSuccess) return e;
    if ((e = prepare_main<TA, TB, 64, false>()) != cudaSuccess) return e;
    if ((e = cudaFuncGetAttributes(&fa, dgemm_mma_tma_kernel<TA, TB, 64, false>)) != cudaSuccess) return e;
    if ((e = prepare_main<TA, TB, 32, false>()) != cudaSuccess) return e;
    if ((e = cudaFuncGetAttributes(&fa, dgemm_mma_tma_kernel<TA, TB, 32, false>)) != cudaSuccess) return e;
    if ((e = prepare_main<TA, TB, 16, false>()) != cudaSuccess) return e;
    return cudaFuncGetAttributes(&fa, dgemm_mma_tma_kernel<TA, TB, 16, false>);
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
    if (tilesM * ((p.N + 15) / 16) >= (1u << 31)) return cudaErrorNotSupported;
    set_last_kernel("dgemm_mma_tma");
    // Widest tile that still gives the 148 SMs about one CTA each; narrower tiles only for
    // problems that 128-wide tiles would leave most SMs idle on.
    const size_t tiles128 = tilesM * ((p.N + 127) / 128), nk = (p.K + BK - 1) / BK;
    // (fewer 128-wide tiles than that but at least 40 K slabs per SM: still 128 wide, shared out by the stream-K kernel)
    const bool share_k = p.tri == TRI_FULL && tiles128 * nk >= (size_t)sm_count() * 40 && gemm_may_allocate() && p.C != p.A && p.C != p.B &&
                         getenv("CLBLAS_B200_NO_STREAMK") == nullptr;
    if (min_bn >= 128 || tiles128 >= 120 || share_k || dgemm_tri_streamk_applies(p)) return launch_t<128>(p, s);
    if (tilesM * ((p.N + 63) / 64) >= 120) return launch_t<64>(p, s);
    if (tilesM * ((p.N + 31) / 32) >= 120) return launch_t<32>(p, s);
    return launch_t<16>(p, s);
}

cudaError_t dgemm_prepare_all_kernels()
{
    cudaError_t e;
    if ((e = prepare_transposition<false, false>()) != cudaSuccess) return e;
    if ((e = prepare_transposition<false, true>()) != cudaSuccess) return e;
    if ((e = prepare_transposition<true, false>()) != cudaSuccess) return e;
    if ((e = prepare_transposition<true, true>()) != cudaSuccess) return e;
    if (get_tensor_map_encoder() == nullptr) return cudaErrorNotSupported;
    return gemm_simt_load_double_kernels();
}

unsigned dgemm_tma_fault_flag() { return read_wait_timeout_flag(); }

}  // namespace cb200
