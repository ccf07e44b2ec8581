// SGEMM in true FP32 (FFMA), TMA-staged: C = alpha*op(A)*op(B) + beta*C, column-major, for
// operands whose base addresses and leading dimensions are multiples of 16 bytes.
//
// B200 counterpart of the reference's AutoGemm sgemm tile kernels, in particular its best one,
// the hand-tuned 128x128 macro-tile with 8x8 micro-tile
// (src/library/blas/AutoGemm/UserGemmKernelSources/sgemm_Col_NT_B1_MX128_NX128_KX16_src.cpp),
// and of the generator they come from (src/library/blas/AutoGemm/KernelOpenCL.py:13-459).
//
// CTA = 128 x BN tile of C (BN = 128, or 64 for problems too small to give every SM a 128-wide
// tile), K in slabs of 32, 256 threads (16 x 16, an 8 x BN/16 register tile each).
// There is no producer warp: late in every slab one thread (lane 0 of a different warp each slab) refills
// the ring slot that was consumed one slab earlier (two TMA bulk-tensor loads; full/empty mbarriers, bounded
// waits).
// Configurations of the same code:
//   * 3-stage ring, at most 128 registers per thread, TWO CTAs per SM: four warps per SM
//     sub-partition hide each other's shared-memory latency and barrier waits;
//   * 5-stage ring, up to 255 registers, one CTA per SM: for the transpose cases whose 4-k
//     fragments need the registers (K-contiguous operands).
// TMA zero-fills beyond M, N, K, so one launch covers ragged shapes; the epilogue is predicated.
//
// Shared layouts:
//  * M/N-contiguous operand (A for transA=N, B for transB=T): box tile x 32 (k), dense rows;
//    a thread reads float4 per k (rows 4*tx..+3 and 64+4*tx..+3), a warp reads 256 contiguous
//    bytes: conflict free.
//  * K-contiguous operand (A for transA=T, B for transB=N): box 32 (k) x tile, 128-byte rows,
//    SWIZZLE_128B; a thread reads one float4 (4 consecutive k) per row, rows tx + 16*i for A so
//    that the 8 lanes of a quarter warp hit 8 different swizzle phases: conflict free.  B rows are
//    shared by the 16 lanes with equal ty (broadcast).
// When A is M-contiguous the products are issued as packed FP32x2 FMAs (fma.rn.f32x2: two IEEE
// FMAs per instruction, bit-identical to scalar FFMA, half the issue slots): per k, 32 packed FMAs,
// 4 LDS.128 and 8 register moves that duplicate the B values.
#include "common.h"
#include "tma_pipeline.cuh"

#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>

namespace cb200 {

namespace {

constexpr int BM = 128, BK = 32;
constexpr int A_BYTES = BM * BK * 4;                // 16 KB
constexpr int THREADS = 256;
constexpr int GROUP_M = 16;

// CTAs per wave as the kernels' `wave` argument (every other wave walks K backwards), or 0 = all forwards when
// CLBLAS_B200_REVERSE_K=0 (a measuring switch).
static unsigned reverse_wave(int ctas) {
    static const bool off = [] { const char* e = getenv("CLBLAS_B200_REVERSE_K"); return e && e[0] == '0'; }();
    return off ? 0u : (unsigned)ctas;
}
constexpr int REFILL_KC = 6;                         // eighth of the slab (0..7) in which the freed slot is refilled

constexpr int stage_bytes(int bn) { return A_BYTES + bn * BK * 4; }
constexpr int smem_bytes(int stages, int bn) { return stages * stage_bytes(bn) + 1024 + 256; }

__device__ __forceinline__ unsigned long long pack2(float lo, float hi)
{
    unsigned long long r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack2(unsigned long long v, float& lo, float& hi)
{
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
// d = a * b + c on both halves (packed FP32x2 FMA of sm_100)
__device__ __forceinline__ unsigned long long ffma2(unsigned long long a, unsigned long long b, unsigned long long c)
{
    unsigned long long d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}

// TRI: compiled-in support for the triangular update (SYRK); without it `tri` is ignored and the epilogue carries
// no per-entry mask.
template <bool TA, bool TB, int BN, int STAGES, int MIN_CTAS, bool TRI>
__global__ void __launch_bounds__(THREADS, MIN_CTAS)
sgemm_ffma_tma_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB,
                      float* __restrict__ C, size_t ldc, size_t M, size_t N, size_t K, float alpha, float beta,
                      unsigned tilesM, unsigned tilesN, unsigned wave, int tri_arg, unsigned splits, size_t split_stride,
                      float* __restrict__ planes, size_t ldw, unsigned* __restrict__ tickets)
{
    int tri = TRI ? tri_arg : TRI_FULL;
    __shared__ unsigned s_ticket;
    constexpr int STAGE_BYTES = stage_bytes(BN);
    constexpr int NJ = BN / 16;                     // columns per thread: 8 or 4
    constexpr int NH = NJ / 4;                      // 4-column groups per thread (64 columns apart)
    constexpr int B_ROW = BN * 4;                   // bytes per k row of an N-contiguous B slab

    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
    uint64_t* empty = full + STAGES;
    pdl_launch_dependents();

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
    // Split-K launches (gridDim.y = splits): this CTA owns K slabs [kt0, kt0 + nk) and writes its partial tile
    // into plane blockIdx.y of a workspace; the CTA of a tile that finishes last sums the planes in plane order
    // (a fixed order, whoever finishes last) and writes C.
    const int nk_total = (int)((K + BK - 1) / BK);
    const int nk_per = (nk_total + (int)splits - 1) / (int)splits;
    const int kt0 = (int)blockIdx.y * nk_per;
    const int nk = max(0, min(nk_per, nk_total - kt0));
    // Every other wave of CTAs walks K backwards: it starts on the K range the wave before it
    // finished on, which is what L2 still holds, instead of re-streaming those panels from DRAM.
    const bool reverse_k = wave != 0 && ((blockIdx.x / wave) & 1);
    const int lane = threadIdx.x % 32;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], THREADS / 32);
        }
        mbar_fence_init();
    }
    __syncthreads();
    pdl_wait();               // everything below reads or writes global memory

    auto issue = [&](int kt) {
        const int s = kt % STAGES;
        unsigned char* sa = smem + s * STAGE_BYTES;
        unsigned char* sb = sa + A_BYTES;
        mbar_expect_tx(&full[s], STAGE_BYTES);
        const int k0 = (kt0 + (reverse_k ? nk - 1 - kt : kt)) * BK;
        if (TA) tma_load_2d(sa, &mapA, k0, (int)m0, &full[s]); else tma_load_2d(sa, &mapA, (int)m0, k0, &full[s]);
        if (TB) tma_load_2d(sb, &mapB, (int)n0, k0, &full[s]); else tma_load_2d(sb, &mapB, k0, (int)n0, &full[s]);
    };
    if (threadIdx.x == 0) {
        tma_prefetch_descriptor(&mapA);
        tma_prefetch_descriptor(&mapB);
        for (int kt = 0; kt < STAGES - 1 && kt < nk; kt++) issue(kt);
    }

    const int tid = threadIdx.x;
    const int tx = tid % 16, ty = tid / 16;

    // Row i (0..7) of this thread's register tile is tile row rowA(i); column j is tile column colB(j).
    auto rowA = [&](int i) { return TA ? tx + 16 * i : tx * 4 + (i & 3) + 64 * (i >> 2); };
    auto colB = [&](int j) { return ty * 4 + (j & 3) + 64 * (j >> 2); };

    // Accumulators.  When A is M-contiguous a 16-byte fragment load delivers rows in adjacent pairs, so
    // the products are packed: acc2[p][j] = rows (2p, 2p+1) of column j.
    float acc[8][NJ];
    unsigned long long acc2[4][NJ];
#pragma unroll
    for (int i = 0; i < 8; i++)
#pragma unroll
        for (int j = 0; j < NJ; j++) {
            if (TA) acc[i][j] = 0.f;
            else if (i < 4) acc2[i][j] = 0ull;
        }

    bool alive = true;
    for (int kt = 0; kt < nk; kt++) {
        const int s = kt % STAGES;
        if (!mbar_wait(&full[s], (kt / STAGES) & 1)) break;
        const unsigned char* sa = smem + s * STAGE_BYTES;
        const unsigned char* sb = sa + A_BYTES;
#pragma unroll
        for (int kc = 0; kc < BK / 4; kc++) {
            // Refill the slot consumed during the previous slab with the slab STAGES-1 ahead.  Done late in
            // this slab (by then even a lagging warp has released that slot) and by a different warp every
            // slab, so that a wait, when there is one, does not always hold back the same warp.
            if (kc == REFILL_KC && threadIdx.x == 32 * (kt & 7) && kt + STAGES - 1 < nk) {
                if (kt >= 1) alive = mbar_wait(&empty[(kt - 1) % STAGES], ((kt - 1) / STAGES) & 1);
                if (alive) issue(kt + STAGES - 1);
            }
            float a4[4][8], b4[4][NJ];
            if (TA) {
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    const float4 v = *reinterpret_cast<const float4*>(sa + (tx + 16 * i) * 128 + ((kc ^ (tx & 7)) << 4));
                    a4[0][i] = v.x; a4[1][i] = v.y; a4[2][i] = v.z; a4[3][i] = v.w;
                }
            }
            if (!TB) {
#pragma unroll
                for (int j = 0; j < NJ; j++) {
                    const int n = ty * 4 + (j & 3) + 64 * (j >> 2);
                    const float4 v = *reinterpret_cast<const float4*>(sb + n * 128 + ((kc ^ (n & 7)) << 4));
                    b4[0][j] = v.x; b4[1][j] = v.y; b4[2][j] = v.z; b4[3][j] = v.w;
                }
            }
#pragma unroll
            for (int q = 0; q < 4; q++) {
                float a[8], b[NJ];
                if (TA) {
#pragma unroll
                    for (int i = 0; i < 8; i++) a[i] = a4[q][i];
                } else {
                    const float4 v0 = *reinterpret_cast<const float4*>(sa + (kc * 4 + q) * 512 + tx * 16);
                    const float4 v1 = *reinterpret_cast<const float4*>(sa + (kc * 4 + q) * 512 + 256 + tx * 16);
                    a[0] = v0.x; a[1] = v0.y; a[2] = v0.z; a[3] = v0.w;
                    a[4] = v1.x; a[5] = v1.y; a[6] = v1.z; a[7] = v1.w;
                }
                if (!TB) {
#pragma unroll
                    for (int j = 0; j < NJ; j++) b[j] = b4[q][j];
                } else {
#pragma unroll
                    for (int h = 0; h < NH; h++) {
                        const float4 v = *reinterpret_cast<const float4*>(sb + (kc * 4 + q) * B_ROW + h * 256 + ty * 16);
                        b[4 * h + 0] = v.x; b[4 * h + 1] = v.y; b[4 * h + 2] = v.z; b[4 * h + 3] = v.w;
                    }
                }
                if (TA) {
#pragma unroll
                    for (int i = 0; i < 8; i++)
#pragma unroll
                        for (int j = 0; j < NJ; j++) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
                } else {
                    unsigned long long a2[4], bd[NJ];
#pragma unroll
                    for (int pr = 0; pr < 4; pr++) a2[pr] = pack2(a[2 * pr], a[2 * pr + 1]);
#pragma unroll
                    for (int j = 0; j < NJ; j++) bd[j] = pack2(b[j], b[j]);
#pragma unroll
                    for (int pr = 0; pr < 4; pr++)
#pragma unroll
                        for (int j = 0; j < NJ; j++) acc2[pr][j] = ffma2(a2[pr], bd[j], acc2[pr][j]);
                }
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[s]);
    }
    if (!TA) {
#pragma unroll
        for (int pr = 0; pr < 4; pr++)
#pragma unroll
            for (int j = 0; j < NJ; j++) unpack2(acc2[pr][j], acc[2 * pr][j], acc[2 * pr + 1][j]);
    }

    // ---- epilogue: D = al*acc + be*D; be == 0 never reads D
    auto epilogue = [&](float* D, size_t ldd, float al, float be, int trimode) {
        const bool useC = (be != 0.f);
        const bool vec = !TA && (!TRI || trimode == TRI_FULL) && ((reinterpret_cast<uintptr_t>(D) & 15) == 0) && (ldd % 4 == 0);
#pragma unroll
        for (int j = 0; j < NJ; j++) {
            const size_t col = n0 + colB(j);
            if (col >= N) continue;
            float* cc = D + col * ldd;
            if (vec) {
#pragma unroll
                for (int h = 0; h < 2; h++) {
                    const size_t row = m0 + tx * 4 + 64 * h;
                    if (row + 3 < M) {
                        float4 r;
                        r.x = al * acc[4 * h + 0][j]; r.y = al * acc[4 * h + 1][j];
                        r.z = al * acc[4 * h + 2][j]; r.w = al * acc[4 * h + 3][j];
                        if (useC) {
                            const float4 o = *reinterpret_cast<const float4*>(cc + row);
                            r.x = fmaf(be, o.x, r.x); r.y = fmaf(be, o.y, r.y);
                            r.z = fmaf(be, o.z, r.z); r.w = fmaf(be, o.w, r.w);
                        }
                        *reinterpret_cast<float4*>(cc + row) = r;
                    } else {
#pragma unroll
                        for (int e = 0; e < 4; e++) {
                            if (row + e < M && !(TRI && tri_masked(trimode, row + e, col))) {
                                float r = al * acc[4 * h + e][j];
                                if (useC) r = fmaf(be, cc[row + e], r);
                                cc[row + e] = r;
                            }
                        }
                    }
                }
            } else {
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    const size_t row = m0 + rowA(i);
                    if (row < M && !(TRI && tri_masked(trimode, row, col))) {
                        float r = al * acc[i][j];
                        if (useC) r = fmaf(be, cc[row], r);
                        cc[row] = r;
                    }
                }
            }
        }
    };
    if (splits <= 1) {
        epilogue(C, ldc, alpha, beta, tri);
        return;
    }
    // ---- split K: partial tile to this CTA's plane, then a ticket; the last CTA of the tile reduces
    epilogue(planes + (size_t)blockIdx.y * split_stride, ldw, 1.f, 0.f, TRI_FULL);
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) s_ticket = atomicAdd(&tickets[blockIdx.x], 1u);
    __syncthreads();
    if (s_ticket != splits - 1) return;
    __threadfence();
#pragma unroll
    for (int i = 0; i < 8; i++)
#pragma unroll
        for (int j = 0; j < NJ; j++) acc[i][j] = 0.f;
    for (unsigned sp = 0; sp < splits; sp++) {
        const float* P = planes + (size_t)sp * split_stride;
#pragma unroll
        for (int j = 0; j < NJ; j++) {
            const size_t col = n0 + colB(j);
            if (col >= N) continue;
            const float* pc = P + col * ldw;
            if (!TA) {
                // ldw is a multiple of 4 and covers the rows up to the next multiple of 4: whole float4s
#pragma unroll
                for (int h = 0; h < 2; h++) {
                    const size_t row = m0 + tx * 4 + 64 * h;
                    if (row < M) {
                        const float4 v = __ldcg(reinterpret_cast<const float4*>(pc + row));
                        acc[4 * h + 0][j] += v.x; acc[4 * h + 1][j] += v.y; acc[4 * h + 2][j] += v.z; acc[4 * h + 3][j] += v.w;
                    }
                }
            } else {
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    const size_t row = m0 + rowA(i);
                    if (row < M) acc[i][j] += __ldcg(pc + row);
                }
            }
        }
    }
    epilogue(C, ldc, alpha, beta, tri);
}

template <bool TA, bool TB, int BN, int STAGES, int MIN_CTAS, bool TRI>
cudaError_t launch(const GemmProblem<float>& p, cudaStream_t s, unsigned splits = 1)
{
    void* enc = get_tensor_map_encoder();
    CUtensorMap mapA, mapB;
    bool ok;
    if (TA) ok = make_tensor_map_2d(&mapA, enc, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, p.A, p.K, p.M, p.lda, BK, BM, CU_TENSOR_MAP_SWIZZLE_128B);
    else    ok = make_tensor_map_2d(&mapA, enc, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, p.A, p.M, p.K, p.lda, BM, BK, CU_TENSOR_MAP_SWIZZLE_NONE);
    if (!ok) return cudaErrorNotSupported;
    if (TB) ok = make_tensor_map_2d(&mapB, enc, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, p.B, p.N, p.K, p.ldb, BN, BK, CU_TENSOR_MAP_SWIZZLE_NONE);
    else    ok = make_tensor_map_2d(&mapB, enc, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, p.B, p.K, p.N, p.ldb, BK, BN, CU_TENSOR_MAP_SWIZZLE_128B);
    if (!ok) return cudaErrorNotSupported;

    constexpr int SMEM = smem_bytes(STAGES, BN);
    static DeviceOnce once;
    cudaError_t e = once.run([] {
        return cudaFuncSetAttribute(sgemm_ffma_tma_kernel<TA, TB, BN, STAGES, MIN_CTAS, TRI>,
                                    cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
    });
    if (e != cudaSuccess) return e;
    const size_t tilesM = (p.M + BM - 1) / BM, tilesN = (p.N + BN - 1) / BN;
    char name[64];
    snprintf(name, sizeof(name), "sgemm_ffma_tma<%c,%c,%d,%d,%d>%s", TA ? 'T' : 'N', TB ? 'T' : 'N', BN, STAGES, MIN_CTAS, TRI ? "+tri" : "");
    float* W = nullptr;
    const size_t ldw = (p.M + 3) / 4 * 4, stride = ldw * p.N, tiles = tilesM * tilesN;
    if (splits > 1 && ws_alloc(reinterpret_cast<void**>(&W), splits * stride * sizeof(float) + tiles * sizeof(unsigned) + 256, s) != cudaSuccess) {
        cudaGetLastError();          // no workspace: the same kernel, unsplit, needs none
        splits = 1;
    }
    if (splits > 1) {
        // partial products into `splits` planes of a workspace; the last CTA of each tile sums them (in plane order) into C
        snprintf(name + strlen(name), sizeof(name) - strlen(name), "+splitk%u", splits);
        set_last_variant(name);
        unsigned* tickets = reinterpret_cast<unsigned*>(W + splits * stride);
        e = cudaMemsetAsync(tickets, 0, tiles * sizeof(unsigned), s);
        if (e == cudaSuccess) {
            e = launch_pdl(sgemm_ffma_tma_kernel<TA, TB, BN, STAGES, MIN_CTAS, TRI>, dim3((unsigned)tiles, splits), dim3(THREADS), SMEM, s,
                           mapA, mapB, p.C, p.ldc, p.M, p.N, p.K, p.alpha, p.beta, (unsigned)tilesM, (unsigned)tilesN, 0u, p.tri, splits, stride,
                           W, ldw, tickets);
            count_launch();
        }
        const cudaError_t e2 = ws_free(W, s);
        return e != cudaSuccess ? e : e2;
    }
    set_last_variant(name);
    e = launch_pdl(sgemm_ffma_tma_kernel<TA, TB, BN, STAGES, MIN_CTAS, TRI>, dim3((unsigned)(tilesM * tilesN)), dim3(THREADS), SMEM, s,
                   mapA, mapB, p.C, p.ldc, p.M, p.N, p.K, p.alpha, p.beta, (unsigned)tilesM, (unsigned)tilesN,
                   reverse_wave(sm_count() * MIN_CTAS), p.tri, 1u, (size_t)0, (float*)nullptr, (size_t)0, (unsigned*)nullptr);
    count_launch();
    return e;
}

// ---------------------------------------------------------------------------------------------
// N/T kernel with a 16 x 8 register tile: 128 x 128 tile of C, 128 threads (8 along M x 16 along N),
// both operands M/N-contiguous (the layout every large SGEMM is repacked into).
//
// Why a second kernel: with the 8 x 8 register tile above, a CTA moves 16 KB from shared memory to
// registers per k-slab row (256 threads x 16 floats), which at 128 B per cycle costs as many cycles as
// the 128 x 128 FMAs themselves -- the profile shows the shared-memory pipe at 83 % next to the FMA
// pipe at 82 %.  A 16 x 8 register tile needs 24 floats per 128 FMAs instead of 16 per 64: 12 KB per
// k row and CTA, 75 % of the FMA time, which leaves the FMA pipe as the only limiter.  The 64 packed
// accumulators take 128 registers, so the budget is 255 registers and two CTAs (eight warps) per SM.
constexpr int T16_THREADS = 128;
constexpr int T16_STAGES = 3;
constexpr int T16_REFILL_KC = 3;        // quarter of the slab (0..3) in which the slot freed one slab earlier is refilled
constexpr int T16_STAGE_BYTES = (128 + 128) * BK * 4;          // 32 KB
constexpr int T16_SMEM = T16_STAGES * T16_STAGE_BYTES + 1024 + 256;

// NCH chunks of eight k rows of the 16 x 8 register tile: sa / sb point at this thread's fragment of the first row in the
// A / B slab in shared memory (512 bytes per k row); `refill` runs once, before chunk REFILL_AT (the producer step of the
// TMA ring).  acc2[2*g + q][4*h + c] = rows (tx*4 + 32*g + 2*q, +1) of column ty*4 + 64*h + c.
template <int NCH, int REFILL_AT, class Refill>
__device__ __forceinline__ void t16_rows(const unsigned char* sa, const unsigned char* sb, unsigned long long (&acc2)[8][8], Refill&& refill)
{
    // Fully unrolled: a trip count of eight k rows keeps the code in the instruction cache but costs 3 % at
    // 8192^3 (fragment loads are not carried across trips), measured.
#pragma unroll
    for (int kc = 0; kc < NCH; kc++) {
        if (kc == REFILL_AT) refill();
#pragma unroll
        for (int q = 0; q < 8; q++) {
            unsigned long long a2[8], bd[8];
#pragma unroll
            for (int g = 0; g < 4; g++) {
                // 16 bytes = rows (0,1) and (2,3) of the group: already the two packed operands
                const ulonglong2 v = *reinterpret_cast<const ulonglong2*>(sa + (kc * 8 + q) * 512 + g * 128);
                a2[2 * g] = v.x; a2[2 * g + 1] = v.y;
            }
#pragma unroll
            for (int h = 0; h < 2; h++) {
                const float4 v = *reinterpret_cast<const float4*>(sb + (kc * 8 + q) * 512 + h * 256);
                bd[4 * h + 0] = pack2(v.x, v.x); bd[4 * h + 1] = pack2(v.y, v.y);
                bd[4 * h + 2] = pack2(v.z, v.z); bd[4 * h + 3] = pack2(v.w, v.w);
            }
#pragma unroll
            for (int i = 0; i < 8; i++)
#pragma unroll
                for (int j = 0; j < 8; j++) acc2[i][j] = ffma2(a2[i], bd[j], acc2[i][j]);
        }
    }
}

// D = al*acc + be*D on row groups [G0, G1) of the thread's 16 x 8 entries of the tile at (m0, n0); be == 0 never reads D.
template <bool TRI, int G0, int G1>
__device__ __forceinline__ void t16_epilogue(const unsigned long long (&acc2)[8][8], float* D, size_t ldd, float al, float be, int trimode,
                                             size_t m0, size_t n0, size_t M, size_t N, int tx, int ty)
{
    const bool useC = (be != 0.f);
    const bool vec = (!TRI || trimode == TRI_FULL) && ((reinterpret_cast<uintptr_t>(D) & 15) == 0) && (ldd % 4 == 0);
#pragma unroll
    for (int j = 0; j < 8; j++) {
        const size_t col = n0 + ty * 4 + (j & 3) + 64 * (j >> 2);
        if (col >= N) continue;
        float* cc = D + col * ldd;
#pragma unroll
        for (int g = G0; g < G1; g++) {
            const size_t row = m0 + tx * 4 + 32 * g;
            float v[4];
            unpack2(acc2[2 * g][j], v[0], v[1]);
            unpack2(acc2[2 * g + 1][j], v[2], v[3]);
            if (vec && row + 3 < M) {
                float4 r;
                r.x = al * v[0]; r.y = al * v[1]; r.z = al * v[2]; r.w = al * v[3];
                if (useC) {
                    const float4 o = *reinterpret_cast<const float4*>(cc + row);
                    r.x = fmaf(be, o.x, r.x); r.y = fmaf(be, o.y, r.y);
                    r.z = fmaf(be, o.z, r.z); r.w = fmaf(be, o.w, r.w);
                }
                *reinterpret_cast<float4*>(cc + row) = r;
            } else {
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    if (row + e < M && !(TRI && tri_masked(trimode, row + e, col))) {
                        float r = al * v[e];
                        if (useC) r = fmaf(be, cc[row + e], r);
                        cc[row + e] = r;
                    }
                }
            }
        }
    }
}

template <bool TRI>
__global__ void __launch_bounds__(T16_THREADS, 2)
sgemm_nt_16x8_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB,
                     float* __restrict__ C, size_t ldc, size_t M, size_t N, size_t K, float alpha, float beta,
                     unsigned tilesM, unsigned tilesN, unsigned wave, int tri_arg, unsigned splits, size_t split_stride,
                     float* __restrict__ planes, size_t ldw, unsigned* __restrict__ tickets)
{
    int tri = TRI ? tri_arg : TRI_FULL;
    __shared__ unsigned s_ticket;
    constexpr int BN = 128;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + T16_STAGES * T16_STAGE_BYTES);
    uint64_t* empty = full + T16_STAGES;
    pdl_launch_dependents();

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
        if (tri_tile_outside(tri, m0, BM, n0, BN)) return;
        if (tri_tile_inside(tri, m0, BM, n0, BN)) tri = TRI_FULL;
    }
    // Split-K launches (gridDim.y = splits): K slabs [kt0, kt0 + nk) belong to this CTA, see the fix-up at the end.
    const int nk_total = (int)((K + BK - 1) / BK);
    const int nk_per = (nk_total + (int)splits - 1) / (int)splits;
    const int kt0 = (int)blockIdx.y * nk_per;
    const int nk = max(0, min(nk_per, nk_total - kt0));
    const bool reverse_k = wave != 0 && ((blockIdx.x / wave) & 1);
    const int lane = threadIdx.x % 32;

    if (threadIdx.x == 0) {
        for (int s = 0; s < T16_STAGES; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], T16_THREADS / 32);
        }
        mbar_fence_init();
    }
    __syncthreads();
    pdl_wait();               // everything below reads or writes global memory

    auto issue = [&](int kt) {
        const int s = kt % T16_STAGES;
        unsigned char* sa = smem + s * T16_STAGE_BYTES;
        unsigned char* sb = sa + A_BYTES;
        mbar_expect_tx(&full[s], T16_STAGE_BYTES);
        const int k0 = (kt0 + (reverse_k ? nk - 1 - kt : kt)) * BK;
        tma_load_2d(sa, &mapA, (int)m0, k0, &full[s]);
        tma_load_2d(sb, &mapB, (int)n0, k0, &full[s]);
    };
    if (threadIdx.x == 0) {
        tma_prefetch_descriptor(&mapA);
        tma_prefetch_descriptor(&mapB);
        for (int kt = 0; kt < T16_STAGES - 1 && kt < nk; kt++) issue(kt);
    }

    const int tx = threadIdx.x % 8, ty = threadIdx.x / 8;
    // rows tx*4 + 32*g + (0..3), g < 4; columns ty*4 + 64*h + (0..3), h < 2
    // acc2[2*g + q][4*h + c] = rows (tx*4 + 32*g + 2*q, +1) of column ty*4 + 64*h + c
    unsigned long long acc2[8][8];
#pragma unroll
    for (int i = 0; i < 8; i++)
#pragma unroll
        for (int j = 0; j < 8; j++) acc2[i][j] = 0ull;

    const int offA = tx * 16, offB = ty * 16;
    bool alive = true;
    for (int kt = 0; kt < nk; kt++) {
        const int s = kt % T16_STAGES;
        if (!mbar_wait(&full[s], (kt / T16_STAGES) & 1)) break;
        const unsigned char* sa = smem + s * T16_STAGE_BYTES + offA;
        const unsigned char* sb = smem + s * T16_STAGE_BYTES + A_BYTES + offB;
        // Refill the slot consumed during the previous slab, in the last quarter of this one (by then even a
        // lagging warp has released it) and from a different warp every slab, so that the wait, when there
        // is one, does not always hold back the same quarter of the CTA.  Measured at 8192^3: first quarter /
        // thread 0: 61.7, last quarter / thread 0: 63.3, last quarter / rotating: 63.5 TFLOP/s.
        t16_rows<BK / 8, T16_REFILL_KC>(sa, sb, acc2, [&] {
            if (threadIdx.x == 32 * (kt & 3) && kt + T16_STAGES - 1 < nk) {
                if (kt >= 1) alive = mbar_wait(&empty[(kt - 1) % T16_STAGES], ((kt - 1) / T16_STAGES) & 1);
                if (alive) issue(kt + T16_STAGES - 1);
            }
        });
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[s]);
    }

    auto epilogue = [&](float* D, size_t ldd, float al, float be, int trimode) {
        t16_epilogue<TRI, 0, 4>(acc2, D, ldd, al, be, trimode, m0, n0, M, N, tx, ty);
    };
    if (splits <= 1) {
        epilogue(C, ldc, alpha, beta, tri);
        return;
    }
    // ---- split K: the partial tile goes to this CTA's plane of the workspace; the CTA of a tile that draws the last
    // ticket adds the planes in plane order (a fixed order, whoever comes last) and writes C.  Nobody waits.
    epilogue(planes + (size_t)blockIdx.y * split_stride, ldw, 1.f, 0.f, TRI_FULL);
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) s_ticket = atomicAdd(&tickets[blockIdx.x], 1u);
    __syncthreads();
    if (s_ticket != splits - 1) return;
    __threadfence();
#pragma unroll
    for (int i = 0; i < 8; i++)
#pragma unroll
        for (int j = 0; j < 8; j++) acc2[i][j] = 0ull;
    const unsigned long long ones = pack2(1.f, 1.f);
    for (unsigned sp = 0; sp < splits; sp++) {
        const float* P = planes + (size_t)sp * split_stride;
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const size_t col = n0 + ty * 4 + (j & 3) + 64 * (j >> 2);
            if (col >= N) continue;
#pragma unroll
            for (int g = 0; g < 4; g++) {
                const size_t row = m0 + tx * 4 + 32 * g;
                if (row >= M) continue;
                // ldw is a multiple of 4 that covers the rows up to the next multiple of 4: whole float4s
                const float4 v = __ldcg(reinterpret_cast<const float4*>(P + col * ldw + row));
                acc2[2 * g][j] = ffma2(pack2(v.x, v.y), ones, acc2[2 * g][j]);            // x * 1 + acc: an exact addition
                acc2[2 * g + 1][j] = ffma2(pack2(v.z, v.w), ones, acc2[2 * g + 1][j]);
            }
        }
    }
    epilogue(C, ldc, alpha, beta, tri);
}

template <bool TRI>
cudaError_t launch_nt_16x8(const GemmProblem<float>& p, cudaStream_t s, unsigned splits = 1)
{
    void* enc = get_tensor_map_encoder();
    CUtensorMap mapA, mapB;
    if (!make_tensor_map_2d(&mapA, enc, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, p.A, p.M, p.K, p.lda, BM, BK, CU_TENSOR_MAP_SWIZZLE_NONE))
        return cudaErrorNotSupported;
    if (!make_tensor_map_2d(&mapB, enc, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, p.B, p.N, p.K, p.ldb, 128, BK, CU_TENSOR_MAP_SWIZZLE_NONE))
        return cudaErrorNotSupported;
    static DeviceOnce once;
    cudaError_t e = once.run([] {
        return cudaFuncSetAttribute(sgemm_nt_16x8_kernel<TRI>, cudaFuncAttributeMaxDynamicSharedMemorySize, T16_SMEM);
    });
    if (e != cudaSuccess) return e;
    const size_t tilesM = (p.M + BM - 1) / BM, tilesN = (p.N + 127) / 128, tiles = tilesM * tilesN;
    float* W = nullptr;
    const size_t ldw = (p.M + 3) / 4 * 4, stride = ldw * p.N;
    if (splits > 1 && ws_alloc(reinterpret_cast<void**>(&W), splits * stride * sizeof(float) + tiles * sizeof(unsigned) + 256, s) != cudaSuccess) {
        cudaGetLastError();          // no workspace: unsplit
        splits = 1;
    }
    if (splits > 1) {
        char name[48];
        snprintf(name, sizeof(name), "sgemm_nt_16x8+splitk%u", splits);
        set_last_variant(name);
        unsigned* tickets = reinterpret_cast<unsigned*>(W + splits * stride);
        e = cudaMemsetAsync(tickets, 0, tiles * sizeof(unsigned), s);
        if (e == cudaSuccess) {
            e = launch_pdl(sgemm_nt_16x8_kernel<TRI>, dim3((unsigned)tiles, splits), dim3(T16_THREADS), T16_SMEM, s,
                           mapA, mapB, p.C, p.ldc, p.M, p.N, p.K, p.alpha, p.beta, (unsigned)tilesM, (unsigned)tilesN, 0u, p.tri,
                           splits, stride, W, ldw, tickets);
            count_launch();
        }
        const cudaError_t e2 = ws_free(W, s);
        return e != cudaSuccess ? e : e2;
    }
    set_last_variant(TRI ? "sgemm_nt_16x8+tri" : "sgemm_nt_16x8");
    e = launch_pdl(sgemm_nt_16x8_kernel<TRI>, dim3((unsigned)tiles), dim3(T16_THREADS), T16_SMEM, s,
                   mapA, mapB, p.C, p.ldc, p.M, p.N, p.K, p.alpha, p.beta, (unsigned)tilesM, (unsigned)tilesN,
                   reverse_wave(sm_count() * 2), p.tri, 1u, (size_t)0, (float*)nullptr, (size_t)0, (unsigned*)nullptr);
    count_launch();
    return e;
}

// How the 8 x 8 kernel covers `tiles` 128 x 128 tiles on `sms` SMs that hold `per_sm` CTAs each.  CTAs of equal length
// run in rounds: a full round of per_sm * sms CTAs takes per_sm times a CTA's length; a last round of at most sms CTAs
// runs them alone on their SMs, which costs one CTA's length (a lone eight-warp CTA reaches an SM's full rate:
// 1536^3, 144 tiles, 50.5 TFLOP/s); a last round of more than sms CTAs costs a full round for a fraction of the
// machine -- the wave quantisation.  Three plans, in units of one tile's length on a whole SM:
//   one CTA per tile                rounds(tiles, 1)
//   K cut in s, reduced in-kernel   rounds(s * tiles, 1 / s) * 1.06     (partial tiles, shorter K loops)
//   stream-K                        per_sm * tiles / (per_sm * sms) / 0.92, every CTA at least 8 slabs
// Measured N/T, TFLOP/s, unsplit / best split / stream-K: 1280^3 34.6 / 36.7 / 36.9, 1536^3 50.5 / 47.3 / 48.3,
// 2048^3 48.9 / 51.0 / 51.9, 2560^3 52.2 / 54.0 / 54.2, 3072^3 57.3 / 56.3 / 56.4, 3584^3 52.7 / 58.0 / 57.1,
// 4096^3 59.0 / 58.5 / 57.8.
struct Plan { int kind; unsigned splits; };       // kind 0: one CTA per tile, 1: split K, 2: stream-K
Plan choose_plan_8x8(size_t tiles, size_t K, size_t sms, size_t per_sm, bool may_alloc)
{
    auto rounds = [&](size_t ctas, double len) {
        const size_t full = ctas / (per_sm * sms), rest = ctas % (per_sm * sms);
        return (double)per_sm * len * full + (rest == 0 ? 0.0 : rest <= sms ? len : (double)per_sm * len);
    };
    Plan best{0, 1};
    double best_t = rounds(tiles, 1.0);
    if (!may_alloc) return best;
    for (unsigned sp = 2; sp <= 4; sp++) {
        if (K / sp < 256) break;
        const double t = rounds(tiles * sp, 1.0 / sp) * 1.06;
        if (t < best_t * 0.999) { best_t = t; best = Plan{1, sp}; }
    }
    const size_t nk = (K + BK - 1) / BK;
    if (tiles * nk >= per_sm * sms * 8) {
        const double t = (double)tiles / (double)sms / 0.92;
        if (t < best_t * 0.98) best = Plan{2, 1};
    }
    return best;
}

// ---------------------------------------------------------------------------------------------
// Stream-K form of the 8 x 8 kernel for products of a few waves: all K slabs of all 128 x 128 tiles are one sequence
// of units, cut into equal consecutive shares, one per CTA of a grid that exactly fills the machine (two CTAs per SM;
// one when A is K-contiguous or the shares would be short).  With one CTA per tile the last round of CTAs is as long
// as the others however few tiles it holds (256 tiles on 296 slots: two rounds of time for 1.73 rounds of work, and SMs
// left with one CTA run below their paired rate); here every CTA works the same number of slabs and all finish
// together.  A CTA whose share covers a whole tile writes C directly; otherwise it stores its partial tile in its slot
// of a workspace and draws a ticket from the tile's counter, and the CTA that draws the last ticket adds the slots in
// slot order -- a fixed order, so the result does not depend on who finishes last -- applies alpha and beta and writes
// C.  Nobody waits for anybody: no spin loop besides the bounded mbarrier waits of the TMA ring.  (The FP64 kernel does
// the same for the tail of its grid, dgemm_mma_tma.cu.)
__device__ __forceinline__ void sk_tile_coords(unsigned tile, unsigned tilesM, unsigned tilesN, unsigned& tm, unsigned& tn)
{
    const unsigned per_group = GROUP_M * tilesN;
    const unsigned g = tile / per_group;
    const unsigned first = g * GROUP_M;
    const unsigned rows = min((unsigned)GROUP_M, tilesM - first);
    const unsigned r = tile - g * per_group;
    tm = first + r % rows;
    tn = r / rows;
}

template <bool TA, bool TB, int STAGES, int MIN_CTAS>
__global__ void __launch_bounds__(THREADS, MIN_CTAS)
sgemm_streamk_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB,
                     float* __restrict__ C, size_t ldc, size_t M, size_t N, size_t K, float alpha, float beta,
                     unsigned tilesM, unsigned tilesN, unsigned units, unsigned upc, unsigned maxc,
                     float* __restrict__ ws, unsigned* __restrict__ counters)
{
    constexpr int BN = 128, NJ = 8, NH = 2;
    constexpr int STAGE_BYTES = stage_bytes(BN);
    constexpr int B_ROW = BN * 4;
    __shared__ unsigned s_ticket;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
    uint64_t* empty = full + STAGES;
    pdl_launch_dependents();

    const unsigned nk = (unsigned)((K + BK - 1) / BK);
    const unsigned u0 = blockIdx.x * upc, u1 = min(u0 + upc, units);
    if (u0 >= u1) return;
    const unsigned count_local = u1 - u0;
    const int lane = threadIdx.x % 32;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], THREADS / 32);
        }
        mbar_fence_init();
    }
    __syncthreads();
    pdl_wait();

    // unit i of this CTA = K slab (u0 + i) % nk of tile (u0 + i) / nk
    auto issue = [&](unsigned i) {
        const unsigned u = u0 + i, t = u / nk, kt = u - t * nk;
        unsigned tm, tn;
        sk_tile_coords(t, tilesM, tilesN, tm, tn);
        const int s = (int)(i % STAGES);
        unsigned char* sa = smem + s * STAGE_BYTES;
        unsigned char* sb = sa + A_BYTES;
        mbar_expect_tx(&full[s], STAGE_BYTES);
        const int k0 = (int)(kt * BK), m0 = (int)(tm * BM), n0 = (int)(tn * BN);
        if (TA) tma_load_2d(sa, &mapA, k0, m0, &full[s]); else tma_load_2d(sa, &mapA, m0, k0, &full[s]);
        if (TB) tma_load_2d(sb, &mapB, n0, k0, &full[s]); else tma_load_2d(sb, &mapB, k0, n0, &full[s]);
    };
    if (threadIdx.x == 0) {
        tma_prefetch_descriptor(&mapA);
        tma_prefetch_descriptor(&mapB);
        for (unsigned i = 0; i < (unsigned)(STAGES - 1) && i < count_local; i++) issue(i);
    }

    const int tid = threadIdx.x;
    const int tx = tid % 16, ty = tid / 16;
    auto rowA = [&](int i) { return TA ? tx + 16 * i : tx * 4 + (i & 3) + 64 * (i >> 2); };
    auto colB = [&](int j) { return ty * 4 + (j & 3) + 64 * (j >> 2); };

    float acc[8][NJ];
    unsigned long long acc2[4][NJ];
    auto clear = [&]() {
#pragma unroll
        for (int i = 0; i < 8; i++)
#pragma unroll
            for (int j = 0; j < NJ; j++) {
                if (TA) acc[i][j] = 0.f;
                else if (i < 4) acc2[i][j] = 0ull;
            }
    };
    clear();

    bool alive = true;
    unsigned i = 0;
    while (i < count_local) {
        const unsigned t = (u0 + i) / nk, seg_first = (u0 + i) - t * nk;
        const unsigned seg_end = min(u1, (t + 1) * nk) - u0;             // one past the last local unit of this segment
        for (; i < seg_end; i++) {
            const int s = (int)(i % STAGES);
            if (!mbar_wait(&full[s], (i / STAGES) & 1)) return;           // flagged; this tile stays unwritten
            const unsigned char* sa = smem + s * STAGE_BYTES;
            const unsigned char* sb = sa + A_BYTES;
#pragma unroll
            for (int kc = 0; kc < BK / 4; kc++) {
                // refill the slot consumed during the previous unit with the unit STAGES-1 ahead (see the kernel above)
                if (kc == REFILL_KC && threadIdx.x == 32 * (i & 7) && i + STAGES - 1 < count_local) {
                    if (i >= 1) alive = mbar_wait(&empty[(i - 1) % STAGES], ((i - 1) / STAGES) & 1);
                    if (alive) issue(i + STAGES - 1);
                }
                float a4[4][8], b4[4][NJ];
                if (TA) {
#pragma unroll
                    for (int r = 0; r < 8; r++) {
                        const float4 v = *reinterpret_cast<const float4*>(sa + (tx + 16 * r) * 128 + ((kc ^ (tx & 7)) << 4));
                        a4[0][r] = v.x; a4[1][r] = v.y; a4[2][r] = v.z; a4[3][r] = v.w;
                    }
                }
                if (!TB) {
#pragma unroll
                    for (int j = 0; j < NJ; j++) {
                        const int n = ty * 4 + (j & 3) + 64 * (j >> 2);
                        const float4 v = *reinterpret_cast<const float4*>(sb + n * 128 + ((kc ^ (n & 7)) << 4));
                        b4[0][j] = v.x; b4[1][j] = v.y; b4[2][j] = v.z; b4[3][j] = v.w;
                    }
                }
#pragma unroll
                for (int q = 0; q < 4; q++) {
                    float a[8], b[NJ];
                    if (TA) {
#pragma unroll
                        for (int r = 0; r < 8; r++) a[r] = a4[q][r];
                    } else {
                        const float4 v0 = *reinterpret_cast<const float4*>(sa + (kc * 4 + q) * 512 + tx * 16);
                        const float4 v1 = *reinterpret_cast<const float4*>(sa + (kc * 4 + q) * 512 + 256 + tx * 16);
                        a[0] = v0.x; a[1] = v0.y; a[2] = v0.z; a[3] = v0.w;
                        a[4] = v1.x; a[5] = v1.y; a[6] = v1.z; a[7] = v1.w;
                    }
                    if (!TB) {
#pragma unroll
                        for (int j = 0; j < NJ; j++) b[j] = b4[q][j];
                    } else {
#pragma unroll
                        for (int h = 0; h < NH; h++) {
                            const float4 v = *reinterpret_cast<const float4*>(sb + (kc * 4 + q) * B_ROW + h * 256 + ty * 16);
                            b[4 * h + 0] = v.x; b[4 * h + 1] = v.y; b[4 * h + 2] = v.z; b[4 * h + 3] = v.w;
                        }
                    }
                    if (TA) {
#pragma unroll
                        for (int r = 0; r < 8; r++)
#pragma unroll
                            for (int j = 0; j < NJ; j++) acc[r][j] = fmaf(a[r], b[j], acc[r][j]);
                    } else {
                        unsigned long long a2[4], bd[NJ];
#pragma unroll
                        for (int pr = 0; pr < 4; pr++) a2[pr] = pack2(a[2 * pr], a[2 * pr + 1]);
#pragma unroll
                        for (int j = 0; j < NJ; j++) bd[j] = pack2(b[j], b[j]);
#pragma unroll
                        for (int pr = 0; pr < 4; pr++)
#pragma unroll
                            for (int j = 0; j < NJ; j++) acc2[pr][j] = ffma2(a2[pr], bd[j], acc2[pr][j]);
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[s]);
        }
        if (!TA) {
#pragma unroll
            for (int pr = 0; pr < 4; pr++)
#pragma unroll
                for (int j = 0; j < NJ; j++) unpack2(acc2[pr][j], acc[2 * pr][j], acc[2 * pr + 1][j]);
        }

        // ---- end of this CTA's segment [seg_first, seg_last] of tile t
        const unsigned seg_last = (u0 + seg_end - 1) - t * nk;
        unsigned tm, tn;
        sk_tile_coords(t, tilesM, tilesN, tm, tn);
        const size_t m0 = (size_t)tm * BM, n0 = (size_t)tn * BN;
        bool write_c = true;
        if (!(seg_first == 0 && seg_last == nk - 1)) {
            const unsigned first_cta = (t * nk) / upc;
            const unsigned idx = blockIdx.x - first_cta;
            const unsigned count = ((t + 1) * nk - 1) / upc - first_cta + 1;
            float* slot = ws + ((size_t)t * maxc + idx) * (size_t)(BM * BN);
#pragma unroll
            for (int r = 0; r < 8; r++)
#pragma unroll
                for (int j = 0; j < NJ; j++) __stcg(slot + (r * NJ + j) * THREADS + tid, acc[r][j]);
            __threadfence();
            __syncthreads();
            if (tid == 0) s_ticket = atomicAdd(&counters[t], 1u);
            __syncthreads();
            write_c = (s_ticket == count - 1);
            if (write_c) {
                __threadfence();
                const float* base = ws + (size_t)t * maxc * (size_t)(BM * BN) + tid;
#pragma unroll
                for (int r = 0; r < 8; r++)
#pragma unroll
                    for (int j = 0; j < NJ; j++) acc[r][j] = 0.f;
                for (unsigned c = 0; c < count; c++) {
                    const float* sl = base + (size_t)c * (BM * BN);
                    float v[8][NJ];
#pragma unroll
                    for (int r = 0; r < 8; r++)
#pragma unroll
                        for (int j = 0; j < NJ; j++) v[r][j] = __ldcg(sl + (r * NJ + j) * THREADS);
#pragma unroll
                    for (int r = 0; r < 8; r++)
#pragma unroll
                        for (int j = 0; j < NJ; j++) acc[r][j] += v[r][j];
                }
            }
            __syncthreads();                                  // s_ticket is reused by the next segment
        }
        if (write_c) {
            // C = alpha*acc + beta*C; beta == 0 never reads C
            const bool useC = (beta != 0.f);
            const bool vec = !TA && ((reinterpret_cast<uintptr_t>(C) & 15) == 0) && (ldc % 4 == 0);
#pragma unroll
            for (int j = 0; j < NJ; j++) {
                const size_t col = n0 + colB(j);
                if (col >= N) continue;
                float* cc = C + col * ldc;
                if (vec) {
#pragma unroll
                    for (int h = 0; h < 2; h++) {
                        const size_t row = m0 + tx * 4 + 64 * h;
                        if (row + 3 < M) {
                            float4 r;
                            r.x = alpha * acc[4 * h + 0][j]; r.y = alpha * acc[4 * h + 1][j];
                            r.z = alpha * acc[4 * h + 2][j]; r.w = alpha * acc[4 * h + 3][j];
                            if (useC) {
                                const float4 o = *reinterpret_cast<const float4*>(cc + row);
                                r.x = fmaf(beta, o.x, r.x); r.y = fmaf(beta, o.y, r.y);
                                r.z = fmaf(beta, o.z, r.z); r.w = fmaf(beta, o.w, r.w);
                            }
                            *reinterpret_cast<float4*>(cc + row) = r;
                        } else {
#pragma unroll
                            for (int e = 0; e < 4; e++) {
                                if (row + e < M) {
                                    float r = alpha * acc[4 * h + e][j];
                                    if (useC) r = fmaf(beta, cc[row + e], r);
                                    cc[row + e] = r;
                                }
                            }
                        }
                    }
                } else {
#pragma unroll
                    for (int r8 = 0; r8 < 8; r8++) {
                        const size_t row = m0 + rowA(r8);
                        if (row < M) {
                            float r = alpha * acc[r8][j];
                            if (useC) r = fmaf(beta, cc[row], r);
                            cc[row] = r;
                        }
                    }
                }
            }
        }
        clear();
    }
}

// ---------------------------------------------------------------------------------------------
// Stream-K with the 16 x 8 register tile on eight-warp CTAs, one CTA per SM, both operands M/N-contiguous.
//
// The 16 x 8 tile needs the 255-register budget, i.e. at most eight warps per SM; as two four-warp CTAs per SM (the
// kernel above) that only pays with many rounds of CTAs.  Here one CTA holds all eight warps: warps 0-3 take k rows
// 0-15 of every slab, warps 4-7 rows 16-31, each group with the full 128 x 128 tile in registers.  At the end of a
// segment (this CTA's run of slabs of one tile) the groups swap halves through shared memory -- group 0 keeps row groups
// 0-1 and receives group 1's sums for them, group 1 keeps row groups 2-3 -- and each finishes its half: straight to C
// when the segment is the whole tile, else to the CTA's slot of the workspace, ticket, and the CTA that draws the last
// ticket adds the slots in slot order (a fixed order) and writes C.  Nobody waits for anybody.
// TRI: a triangular update (SYRK, HERK): the tiles are those that touch the triangle, in the order of tri_tile_coords, and
// tiles on the diagonal mask their stores.
constexpr int T16W_THREADS = 256;
constexpr int T16W_STAGES = 4;
constexpr int T16W_RED_BYTES = 64 * 128 * 8;         // the halves the two groups hand each other
constexpr int T16W_SMEM = T16W_STAGES * T16_STAGE_BYTES + T16W_RED_BYTES + 1024 + 256;
constexpr size_t T16W_MIN_UNITS = 8;                  // smallest share of a CTA, in K slabs of 32

template <bool TRI>
__global__ void __launch_bounds__(T16W_THREADS, 1)
sgemm_nt_16x8w_streamk_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB,
                              float* __restrict__ C, size_t ldc, size_t M, size_t N, size_t K, float alpha, float beta,
                              unsigned tilesM, unsigned tilesN, unsigned units, unsigned upc, int tri,
                              unsigned long long* __restrict__ ws, unsigned* __restrict__ counters)
{
    __shared__ unsigned s_ticket;
    __shared__ unsigned s_tile[3];             // TRI: the tile the producer looked up last, and its coordinates
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    unsigned long long* red = reinterpret_cast<unsigned long long*>(smem + T16W_STAGES * T16_STAGE_BYTES);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + T16W_STAGES * T16_STAGE_BYTES + T16W_RED_BYTES);
    uint64_t* empty = full + T16W_STAGES;
    pdl_launch_dependents();

    const unsigned nk = (unsigned)((K + BK - 1) / BK);
    const unsigned u0 = blockIdx.x * upc, u1 = min(u0 + upc, units);
    if (u0 >= u1) return;
    const unsigned count_local = u1 - u0;
    const int lane = threadIdx.x % 32;

    if (threadIdx.x == 0) {
        for (int s = 0; s < T16W_STAGES; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], T16W_THREADS / 32);
        }
        mbar_fence_init();
        s_tile[0] = 0xffffffffu;
    }
    __syncthreads();
    pdl_wait();

    auto tile_coords = [&](unsigned t, unsigned& tm, unsigned& tn) {
        if (TRI) tri_tile_coords(tri, t, tilesM, tilesN, tm, tn);
        else sk_tile_coords(t, tilesM, tilesN, tm, tn);
    };
    // unit i of this CTA = K slab (u0 + i) % nk of tile (u0 + i) / nk
    auto issue = [&](unsigned i) {
        const unsigned u = u0 + i, t = u / nk, kt = u - t * nk;
        unsigned tm, tn;
        if (TRI) {
            // The look-up walks the tile columns; it is done once per tile and kept for the next K slabs.  The producers of
            // consecutive slabs are different threads, ordered by the empty barrier each of them waits on first.
            if (s_tile[0] != t) { tile_coords(t, tm, tn); s_tile[0] = t; s_tile[1] = tm; s_tile[2] = tn; }
            else { tm = s_tile[1]; tn = s_tile[2]; }
        } else {
            tile_coords(t, tm, tn);
        }
        const int s = (int)(i % T16W_STAGES);
        unsigned char* sa = smem + s * T16_STAGE_BYTES;
        unsigned char* sb = sa + A_BYTES;
        mbar_expect_tx(&full[s], T16_STAGE_BYTES);
        tma_load_2d(sa, &mapA, (int)(tm * BM), (int)(kt * BK), &full[s]);
        tma_load_2d(sb, &mapB, (int)(tn * 128), (int)(kt * BK), &full[s]);
    };
    if (threadIdx.x == 0) {
        tma_prefetch_descriptor(&mapA);
        tma_prefetch_descriptor(&mapB);
        for (unsigned i = 0; i < (unsigned)(T16W_STAGES - 1) && i < count_local; i++) issue(i);
    }

    const int tid = threadIdx.x, grp = tid / 128, tg = tid % 128, tx = tg % 8, ty = tg / 8;
    unsigned long long acc2[8][8];
    auto clear = [&]() {
#pragma unroll
        for (int i = 0; i < 8; i++)
#pragma unroll
            for (int j = 0; j < 8; j++) acc2[i][j] = 0ull;
    };
    clear();

    const int offA = grp * (16 * 512) + tx * 16, offB = A_BYTES + grp * (16 * 512) + ty * 16;
    const unsigned long long ones = pack2(1.f, 1.f);
    bool alive = true;
    unsigned i = 0;
    while (i < count_local) {
        const unsigned t = (u0 + i) / nk, seg_first = (u0 + i) - t * nk;
        const unsigned seg_end = min(u1, (t + 1) * nk) - u0;              // one past the last local unit of this segment
        const bool first_seg = (i == 0);
        for (; i < seg_end; i++) {
            const int s = (int)(i % T16W_STAGES);
            if (!mbar_wait(&full[s], (i / T16W_STAGES) & 1)) return;      // flagged; this tile stays unwritten
            const unsigned char* sa = smem + s * T16_STAGE_BYTES + offA;
            const unsigned char* sb = smem + s * T16_STAGE_BYTES + offB;
            // the slot freed one slab earlier is refilled in the second half of this one, by a different warp every slab
            t16_rows<2, 1>(sa, sb, acc2, [&] {
                if (threadIdx.x == 32 * (i & 7) && i + T16W_STAGES - 1 < count_local) {
                    if (i >= 1) alive = mbar_wait(&empty[(i - 1) % T16W_STAGES], ((i - 1) / T16W_STAGES) & 1);
                    if (alive) issue(i + T16W_STAGES - 1);
                }
            });
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[s]);
        }

        // ---- end of this CTA's segment [seg_first, seg_last] of tile t: the groups swap halves ...
        {
            unsigned long long* out = red + (size_t)(grp * 32) * 128 + tg;
#pragma unroll
            for (int r = 0; r < 4; r++)
#pragma unroll
                for (int j = 0; j < 8; j++) out[(r * 8 + j) * 128] = grp == 0 ? acc2[4 + r][j] : acc2[r][j];
        }
        __syncthreads();
        {
            const unsigned long long* in = red + (size_t)((1 - grp) * 32) * 128 + tg;
#pragma unroll
            for (int r = 0; r < 4; r++)
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    const unsigned long long v = in[(r * 8 + j) * 128];
                    if (grp == 0) acc2[r][j] = ffma2(v, ones, acc2[r][j]);            // x * 1 + acc: an exact addition
                    else acc2[4 + r][j] = ffma2(v, ones, acc2[4 + r][j]);
                }
        }
        // ... and each finishes its own: acc2[0..3] (row groups 0-1) in group 0, acc2[4..7] (row groups 2-3) in group 1
        const unsigned seg_last = (u0 + seg_end - 1) - t * nk;
        unsigned tm, tn;
        tile_coords(t, tm, tn);
        const size_t m0 = (size_t)tm * BM, n0 = (size_t)tn * 128;
        bool write_c = true;
        if (!(seg_first == 0 && seg_last == nk - 1)) {
            // Two slots per CTA: a partial tile is either the CTA's first segment (slot 0) or, begun at a tile boundary and
            // cut short by the end of the share, its last (slot 1); whole tiles in between need none.
            const unsigned first_cta = (t * nk) / upc;
            const unsigned count = ((t + 1) * nk - 1) / upc - first_cta + 1;
            unsigned long long* slot = ws + ((size_t)blockIdx.x * 2 + (first_seg ? 0 : 1)) * (size_t)(32 * T16W_THREADS);
#pragma unroll
            for (int r = 0; r < 4; r++)
#pragma unroll
                for (int j = 0; j < 8; j++) __stcg(slot + (r * 8 + j) * T16W_THREADS + tid, grp == 0 ? acc2[r][j] : acc2[4 + r][j]);
            __threadfence();
            __syncthreads();
            if (tid == 0) s_ticket = atomicAdd(&counters[t], 1u);
            __syncthreads();
            write_c = (s_ticket == count - 1);
            if (write_c) {
                __threadfence();
                unsigned long long sum[4][8];
#pragma unroll
                for (int r = 0; r < 4; r++)
#pragma unroll
                    for (int j = 0; j < 8; j++) sum[r][j] = 0ull;
                for (unsigned c = first_cta; c < first_cta + count; c++) {
                    // CTA c's part of this tile is its first segment if its share starts inside the tile
                    const unsigned long long* sl = ws + ((size_t)c * 2 + (c * upc >= t * nk ? 0 : 1)) * (size_t)(32 * T16W_THREADS) + tid;
                    unsigned long long v[4][8];               // thirty-two independent loads in flight
#pragma unroll
                    for (int r = 0; r < 4; r++)
#pragma unroll
                        for (int j = 0; j < 8; j++) v[r][j] = __ldcg(sl + (r * 8 + j) * T16W_THREADS);
#pragma unroll
                    for (int r = 0; r < 4; r++)
#pragma unroll
                        for (int j = 0; j < 8; j++) sum[r][j] = ffma2(v[r][j], ones, sum[r][j]);
                }
#pragma unroll
                for (int r = 0; r < 4; r++)
#pragma unroll
                    for (int j = 0; j < 8; j++) {
                        if (grp == 0) acc2[r][j] = sum[r][j]; else acc2[4 + r][j] = sum[r][j];
                    }
            }
        }
        if (write_c) {
            const int trimode = TRI && !tri_tile_inside(tri, m0, BM, n0, 128) ? tri : TRI_FULL;     // tiles on the diagonal mask their stores
            if (grp == 0) t16_epilogue<TRI, 0, 2>(acc2, C, ldc, alpha, beta, trimode, m0, n0, M, N, tx, ty);
            else t16_epilogue<TRI, 2, 4>(acc2, C, ldc, alpha, beta, trimode, m0, n0, M, N, tx, ty);
        }
        __syncthreads();                                      // the exchange buffer and s_ticket are reused by the next segment
        clear();
    }
}

template <bool TRI>
cudaError_t launch_nt_16x8w_streamk(const GemmProblem<float>& p, cudaStream_t s)
{
    void* enc = get_tensor_map_encoder();
    CUtensorMap mapA, mapB;
    if (!make_tensor_map_2d(&mapA, enc, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, p.A, p.M, p.K, p.lda, BM, BK, CU_TENSOR_MAP_SWIZZLE_NONE))
        return cudaErrorNotSupported;
    if (!make_tensor_map_2d(&mapB, enc, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, p.B, p.N, p.K, p.ldb, 128, BK, CU_TENSOR_MAP_SWIZZLE_NONE))
        return cudaErrorNotSupported;
    static DeviceOnce once;
    cudaError_t e = once.run([] {
        return cudaFuncSetAttribute(sgemm_nt_16x8w_streamk_kernel<TRI>, cudaFuncAttributeMaxDynamicSharedMemorySize, T16W_SMEM);
    });
    if (e != cudaSuccess) return e;
    const size_t tilesM = (p.M + BM - 1) / BM, tilesN = (p.N + 127) / 128, tiles = tri_tile_count(TRI ? p.tri : TRI_FULL, tilesM, tilesN);
    if (tiles == 0) return cudaSuccess;
    const size_t nk = (p.K + BK - 1) / BK, units = tiles * nk;
    if (units >= (1ull << 31)) return cudaErrorNotSupported;
    const size_t ctas = std::max<size_t>(1, std::min<size_t>((size_t)sm_count(), units / T16W_MIN_UNITS));
    const size_t upc = (units + ctas - 1) / ctas, grid = (units + upc - 1) / upc;
    const size_t ws_words = grid * 2 * (size_t)(32 * T16W_THREADS);               // two partial-tile slots per CTA
    unsigned long long* ws = nullptr;
    e = ws_alloc(reinterpret_cast<void**>(&ws), ws_words * sizeof(unsigned long long) + tiles * sizeof(unsigned) + 256, s);
    if (e != cudaSuccess) { cudaGetLastError(); return cudaErrorNotSupported; }     // the caller goes on to a kernel that needs no workspace
    unsigned* counters = reinterpret_cast<unsigned*>(ws + ws_words);
    e = cudaMemsetAsync(counters, 0, tiles * sizeof(unsigned), s);
    if (e == cudaSuccess) {
        set_last_variant(TRI ? "sgemm_nt_16x8w_streamk+tri" : "sgemm_nt_16x8w_streamk");
        e = launch_pdl(sgemm_nt_16x8w_streamk_kernel<TRI>, dim3((unsigned)grid), dim3(T16W_THREADS), T16W_SMEM, s,
                       mapA, mapB, p.C, p.ldc, p.M, p.N, p.K, p.alpha, p.beta, (unsigned)tilesM, (unsigned)tilesN, (unsigned)units,
                       (unsigned)upc, p.tri, ws, counters);
        count_launch();
    }
    const cudaError_t e2 = ws_free(ws, s);
    return e != cudaSuccess ? e : e2;
}

constexpr unsigned SK_MIN_UNITS = 4;         // smallest share of a CTA, in K slabs of 32
constexpr unsigned SK_PAIR_MIN_UNITS = 20;   // smallest share for which two CTAs per SM beat one

template <bool TA, bool TB, int STAGES, int MIN_CTAS>
cudaError_t launch_streamk(const GemmProblem<float>& p, cudaStream_t s)
{
    void* enc = get_tensor_map_encoder();
    CUtensorMap mapA, mapB;
    bool ok;
    if (TA) ok = make_tensor_map_2d(&mapA, enc, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, p.A, p.K, p.M, p.lda, BK, BM, CU_TENSOR_MAP_SWIZZLE_128B);
    else    ok = make_tensor_map_2d(&mapA, enc, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, p.A, p.M, p.K, p.lda, BM, BK, CU_TENSOR_MAP_SWIZZLE_NONE);
    if (!ok) return cudaErrorNotSupported;
    if (TB) ok = make_tensor_map_2d(&mapB, enc, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, p.B, p.N, p.K, p.ldb, 128, BK, CU_TENSOR_MAP_SWIZZLE_NONE);
    else    ok = make_tensor_map_2d(&mapB, enc, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, p.B, p.K, p.N, p.ldb, BK, 128, CU_TENSOR_MAP_SWIZZLE_128B);
    if (!ok) return cudaErrorNotSupported;
    constexpr int SMEM = smem_bytes(STAGES, 128);
    static DeviceOnce once;
    cudaError_t e = once.run([] {
        return cudaFuncSetAttribute(sgemm_streamk_kernel<TA, TB, STAGES, MIN_CTAS>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
    });
    if (e != cudaSuccess) return e;
    const size_t tilesM = (p.M + BM - 1) / BM, tilesN = (p.N + 127) / 128, tiles = tilesM * tilesN;
    const size_t nk = (p.K + BK - 1) / BK, units = tiles * nk;
    if (units >= (1ull << 31)) return cudaErrorNotSupported;
    // Two CTAs per SM only when each still gets 20 slabs: shorter shares are mostly fixed cost (pipeline fill, partial-tile
    // store, reduction), and one CTA per SM with a share twice as long wins (N/T, TFLOP/s, one / two per SM: 1152^3 38.1 /
    // 36.2, 1280^3 41.5 / 37.3, 1408^3 45.6 / 44.6, but 1536^3 47.9 / 48.4, 2048^3 51.7 / 52.0).
    size_t slots = (size_t)sm_count() * MIN_CTAS;
    if (MIN_CTAS > 1 && units < slots * SK_PAIR_MIN_UNITS) slots = (size_t)sm_count();
    const size_t ctas = std::max<size_t>(1, std::min<size_t>(slots, units / SK_MIN_UNITS));
    const size_t upc = (units + ctas - 1) / ctas;
    const size_t maxc = (nk + upc - 1) / upc + 1;
    const size_t ws_floats = tiles * maxc * (size_t)(BM * 128);
    float* ws = nullptr;
    e = ws_alloc(reinterpret_cast<void**>(&ws), ws_floats * sizeof(float) + tiles * sizeof(unsigned) + 256, s);
    if (e != cudaSuccess) { cudaGetLastError(); return cudaErrorNotSupported; }     // the caller falls back to one CTA per tile
    unsigned* counters = reinterpret_cast<unsigned*>(ws + ws_floats);
    e = cudaMemsetAsync(counters, 0, tiles * sizeof(unsigned), s);
    if (e == cudaSuccess) {
        char name[64];
        snprintf(name, sizeof(name), "sgemm_streamk<%c,%c>", TA ? 'T' : 'N', TB ? 'T' : 'N');
        set_last_variant(name);
        e = launch_pdl(sgemm_streamk_kernel<TA, TB, STAGES, MIN_CTAS>, dim3((unsigned)((units + upc - 1) / upc)), dim3(THREADS), SMEM, s,
                       mapA, mapB, p.C, p.ldc, p.M, p.N, p.K, p.alpha, p.beta, (unsigned)tilesM, (unsigned)tilesN, (unsigned)units,
                       (unsigned)upc, (unsigned)maxc, ws, counters);
        count_launch();
    }
    const cudaError_t e2 = ws_free(ws, s);
    return e != cudaSuccess ? e : e2;
}

cudaError_t launch_streamk_any(const GemmProblem<float>& p, cudaStream_t s)
{
    if (!p.ta && !p.tb) return launch_streamk<false, false, 3, 2>(p, s);
    if (!p.ta && p.tb) return launch_streamk<false, true, 3, 2>(p, s);
    if (p.ta && !p.tb) return launch_streamk<true, false, 5, 1>(p, s);
    return launch_streamk<true, true, 5, 1>(p, s);
}

template <int BN, int STAGES, int MIN_CTAS>
cudaError_t launch_any(const GemmProblem<float>& p, cudaStream_t s, unsigned splits = 1)
{
    if (splits > 1) {
        if (!p.ta && !p.tb) return launch<false, false, BN, STAGES, MIN_CTAS, false>(p, s, splits);
        if (!p.ta && p.tb) return launch<false, true, BN, STAGES, MIN_CTAS, false>(p, s, splits);
        if (p.ta && !p.tb) return launch<true, false, BN, STAGES, MIN_CTAS, false>(p, s, splits);
        return launch<true, true, BN, STAGES, MIN_CTAS, false>(p, s, splits);
    }
    if (p.tri != TRI_FULL) {
        if (!p.ta && !p.tb) return launch<false, false, BN, STAGES, MIN_CTAS, true>(p, s);
        if (!p.ta && p.tb) return launch<false, true, BN, STAGES, MIN_CTAS, true>(p, s);
        if (p.ta && !p.tb) return launch<true, false, BN, STAGES, MIN_CTAS, true>(p, s);
        return launch<true, true, BN, STAGES, MIN_CTAS, true>(p, s);
    }
    if (!p.ta && !p.tb) return launch<false, false, BN, STAGES, MIN_CTAS, false>(p, s);
    if (!p.ta && p.tb) return launch<false, true, BN, STAGES, MIN_CTAS, false>(p, s);
    if (p.ta && !p.tb) return launch<true, false, BN, STAGES, MIN_CTAS, false>(p, s);
    return launch<true, true, BN, STAGES, MIN_CTAS, false>(p, s);
}

}  // namespace

cudaError_t launch_sgemm_ffma_tma(const GemmProblem<float>& p, cudaStream_t s, int min_bn)
{
    if (!aligned16(p.A) || !aligned16(p.B) || (p.lda & 3) || (p.ldb & 3)) return cudaErrorNotSupported;
    if (p.M >= (1u << 31) || p.N >= (1u << 31) || p.K >= (1u << 31)) return cudaErrorNotSupported;
    const size_t tilesM = (p.M + BM - 1) / BM;
    const size_t tiles128 = tilesM * ((p.N + 127) / 128);
    if (tilesM * ((p.N + 63) / 64) >= (1u << 31)) return cudaErrorNotSupported;
    set_last_kernel("sgemm_ffma_tma");
    const int forced = forced_gemm_path();
    if (forced == PATH_TMA_ONE_CTA) return launch_any<128, 5, 1>(p, s);
    if (forced == PATH_TMA_TWO_CTAS) return launch_any<128, 3, 2>(p, s);
    const bool may_split = gemm_may_allocate() && p.C != p.A && p.C != p.B && getenv("CLBLAS_B200_NO_SPLITK") == nullptr;
    // Tuning aid: CLBLAS_B200_SGEMM_FORCE="<tile>,<splits>" with tile 64 / 128 (8 x 8 register-tile kernel), 16 (16 x 8), 18 (16 x 8 on
    // eight-warp CTAs, stream-K) or 1 (8 x 8 stream-K).
    if (const char* f = getenv("CLBLAS_B200_SGEMM_FORCE")) {
        int tile = 0, sp = 1;
        if (sscanf(f, "%d,%d", &tile, &sp) >= 1 && may_split && p.tri == TRI_FULL && min_bn < 128 && sp >= 1 && sp <= 8) {
            if (tile == 16 && !p.ta && p.tb) return launch_nt_16x8<false>(p, s, (unsigned)sp);
            if (tile == 18 && !p.ta && p.tb) { const cudaError_t e = launch_nt_16x8w_streamk<false>(p, s); if (e != cudaErrorNotSupported) return e; }
            if (tile == 1) { const cudaError_t e = launch_streamk_any(p, s); if (e != cudaErrorNotSupported) return e; }     // "1,0": stream-K
            if (tile == 64) return p.ta ? launch_any<64, 5, 1>(p, s, (unsigned)sp) : launch_any<64, 3, 2>(p, s, (unsigned)sp);
            if (tile == 128) return p.ta ? launch_any<128, 5, 1>(p, s, (unsigned)sp) : launch_any<128, 3, 2>(p, s, (unsigned)sp);
        }
    }
    // The 16 x 8 register-tile kernel has four warps per CTA: it needs both of an SM's CTA slots filled for several
    // waves and a K loop long enough to amortise its per-thread epilogue.  Measured against the 8 x 8 kernel: 8192^3
    // 63.5 vs 57.8-60.2, 6144^3 62.2 vs 58.6, 4096^3 58.9 vs 59.0, but 1536^3 (144 tiles) 35.6 vs 50.5, 2048^3 44.5 vs 48.9
    // and 4096 x 4096 x 512 48.7 vs 53.9 TFLOP/s.  From four waves on it takes the unsplit N/T products.
    const bool k8x8 = getenv("CLBLAS_B200_SGEMM_8X8") != nullptr;
    const bool big_nt = !p.ta && p.tb && min_bn < 128 && tiles128 >= (size_t)sm_count() * 4 && p.K >= 1024 && !k8x8;
    const bool c_vec = (reinterpret_cast<uintptr_t>(p.C) & 15) == 0 && p.ldc % 4 == 0;
    const bool share_k = may_split && getenv("CLBLAS_B200_NO_STREAMK") == nullptr && !k8x8;
    // Triangular updates (SYRK, HERK) of N/T form with a K loop of at least 36 slabs: the eight-warp 16 x 8 stream-K kernel
    // over the tiles that touch the triangle.  With one CTA per tile those tiles come in partly filled rounds (order 4096:
    // 528 tiles on 296 slots).
    if (!p.ta && p.tb && p.tri != TRI_FULL && min_bn < 128 && share_k && c_vec && (p.K + BK - 1) / BK >= 36) {
        const size_t tt = tri_tile_count(p.tri, tilesM, (p.N + 127) / 128), nk = (p.K + BK - 1) / BK;
        if (tt <= (size_t)sm_count() * 16 && tt * nk >= (size_t)sm_count() * T16W_MIN_UNITS) {
            const cudaError_t e = launch_nt_16x8w_streamk<true>(p, s);
            if (e != cudaErrorNotSupported) return e;
        }
    }
    if (big_nt && p.tri != TRI_FULL) return launch_nt_16x8<true>(p, s);
    // N/T products of up to sixteen tiles per SM with a K loop of at least 36 slabs: the eight-warp 16 x 8 stream-K kernel.
    // Measured against the choices below (TFLOP/s, this kernel / the best of the others): 1152^3 38.9 / 38.0, 1408^3 47.6 /
    // 45.5, 2048^3 55.2 / 51.1, 2560^3 58.0 / 54.3, 3072^3 59.8 / 57.5, 4096^3 61.4 / 58.9, 5120^3 62.1 / 61.0, 6144^3 62.6 /
    // 62.2, 1024 x 1024 x 8192 57.3 / 52.7, 768 x 768 x 2048 37.7 / 32.7; but 8192^3 62.8 / 63.5, and with short K loops its
    // exposed epilogue (one CTA per SM: nothing else runs meanwhile) loses: 1024^3 33.5 / 33.4, 4096 x 4096 x 1024 53.3 /
    // 53.9, 8192 x 8192 x 1024 54.7 / 58.3, 4096 x 4096 x 256 36.0 / 51.4.
    {
        const size_t nk = (p.K + BK - 1) / BK, sms = (size_t)sm_count();
        // (C must allow 16-byte accesses: the element-wise epilogue is exposed too -- the ragged row-major product with
        // C at an offset of 5 elements ran at 47.2 against 49.1 TFLOP/s with K in two.)
        if (!p.ta && p.tb && p.tri == TRI_FULL && min_bn < 128 && share_k && nk >= 36 && tiles128 <= sms * 16 && c_vec &&
            tiles128 * nk >= sms * T16W_MIN_UNITS) {
            const cudaError_t e = launch_nt_16x8w_streamk<false>(p, s);
            if (e != cudaErrorNotSupported) return e;
        }
    }
    // Between about half a wave and twelve waves the 8 x 8 kernel's rounds may come out uneven: split K or go
    // stream-K where the model says so (choose_plan_8x8).
    if (p.tri == TRI_FULL && min_bn < 128 && p.K >= 256 && tiles128 >= 64 && tiles128 < (size_t)sm_count() * 12) {
        Plan plan = choose_plan_8x8(tiles128, p.K, (size_t)sm_count(), p.ta ? 1 : 2, may_split);
        if (tiles128 < 96 && plan.kind != 2) plan = Plan{0, 1};      // below 96 tiles the 128 x 64 tiles further down beat a split
        // Where the rounds would come out uneven, N/T products with 24 to 35 K slabs are better off with the eight-warp
        // 16 x 8 stream-K kernel than with a split (2048 x 2048 x 1024: 47.4 against 44.1 TFLOP/s, 2560 x 2560 x 1024 49.9 / 45.5,
        // 2048 x 2048 x 768 43.9 / 43.1); where one CTA per tile fills its rounds it is not (3072 x 3072 x 1024: 51.4 / 55.3).
        if (plan.kind != 0 && !p.ta && p.tb && share_k && c_vec && (p.K + BK - 1) / BK >= 24) {
            const cudaError_t e = launch_nt_16x8w_streamk<false>(p, s);
            if (e != cudaErrorNotSupported) return e;
        }
        if (plan.kind == 2) {
            const cudaError_t e = launch_streamk_any(p, s);
            if (e != cudaErrorNotSupported) return e;
        } else if (plan.kind == 1) {
            return p.ta ? launch_any<128, 5, 1>(p, s, plan.splits) : launch_any<128, 3, 2>(p, s, plan.splits);
        }
    }
    if (big_nt) return launch_nt_16x8<false>(p, s);
    // Fewer 128-wide tiles than SMs: halve the tile width so that twice as many CTAs share the work
    // (three of them fit an SM).  With A K-contiguous the 4-k fragments need the one-CTA register budget.
    if (min_bn < 128 && tiles128 < 120) {
        // Tiles for less than a third of the SMs' CTA slots and a long K loop: split K over 2-4 CTAs per tile, partial tiles
        // summed in plane order by the CTA that finishes last (768 x 768 x 2048 N/N: 18.6 -> 34.2 TFLOP/s; with more
        // tiles than that the split loses: 1024^3, 128 tiles, N/T 33.4 unsplit against 29.8 TFLOP/s in two).
        const size_t tiles64 = tilesM * ((p.N + 63) / 64);
        const size_t slots = (size_t)sm_count() * (p.ta ? 1 : 2);
        unsigned splits = 1;
        if (p.tri == TRI_FULL && tiles64 * 3 <= slots && may_split)
            splits = (unsigned)std::max<size_t>(1, std::min<size_t>(std::min<size_t>(4, slots / tiles64), p.K / 256));
        if (p.ta) return launch_any<64, 5, 1>(p, s, splits);
        return launch_any<64, 3, 2>(p, s, splits);
    }
    // A K-contiguous operand is fetched 4 k at a time (32 fragment registers on top of the
    // accumulators), which the two-CTA budget of 128 registers holds only for B; measured at 8192^3
    // with packed FMAs: N/T 60.2 (two CTAs) vs 53.6 TFLOP/s (one), N/N 48.6 vs 47.2.
    if (!p.ta) return launch_any<128, 3, 2>(p, s);
    return launch_any<128, 5, 1>(p, s);
}

unsigned sgemm_tma_fault_flag() { return read_wait_timeout_flag(); }

}  // namespace cb200
