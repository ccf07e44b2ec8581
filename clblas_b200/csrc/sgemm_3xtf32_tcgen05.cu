// Optional SGEMM variant on the 5th-generation tensor cores: every FP32 operand is split into two
// TF32 numbers (x = hi + lo, hi = rn_tf32(x), lo = rn_tf32(x - hi)) and the product is formed as
// lo*hi + hi*lo + hi*hi with FP32 accumulation in tensor memory ("3xTF32").  The dropped lo*lo term and
// the residual of the split are of relative size 2^-22, far inside the 4*K*u bound (u = 2^-24) the
// library's SGEMM is held to, but the result is NOT bit-identical to an FFMA evaluation, so this path
// is opt-in (clblasB200SetGemmPath(4)); the default SGEMM stays the true-FP32 FFMA kernel.
// The reference has no counterpart (its sgemm kernels are scalar mad() code,
// src/library/blas/AutoGemm/KernelOpenCL.py:171-181).
//
// CTA = 128 x 256 tile of C, K in slabs of 16 (64-byte swizzled rows), ring of 5 slabs, 10 warps:
//   warp 0    producer: TMA loads of the A and B slabs (both K-contiguous, SWIZZLE_64B), issued
//             four slabs ahead of the tensor core;
//   warp 1    owns tensor memory (tcgen05.alloc / dealloc: 256 accumulator columns + a ring of A
//             operands) and issues the MMAs: per 8-wide k step three tcgen05.mma.kind::tf32
//             (M=128, N=256, K=8), B through shared-memory descriptors, A from tensor memory;
//             tcgen05.commit releases the ring slot and, at the end, publishes the accumulator;
//   warps 2-9 splitters: hi is the raw FP32 word itself (the tensor core truncates it); lo is computed
//             with integer adds and masks (the conversion instruction is a quarter-rate pipe).  B lo
//             is written next to the raw slab in the same swizzled layout (element-wise, layout
//             agnostic); A hi and lo go to tensor memory with tcgen05.st (warps 2-5, one row per
//             thread).  fence.proxy.async + tcgen05 fences hand the slot to warp 1.  After the last
//             slab the same warps are the epilogue: tcgen05.ld of their
//             quarter of the 128 accumulator lanes (two warps share a quarter, half the columns each),
//             alpha/beta, coalesced stores.
// Every wait is bounded; all roles meet at one barrier before tensor memory is freed.
// Operands that are not K-contiguous (A for transA=N, B for transB=T) or not 16-byte aligned are
// transposed / copied into a workspace first (repack.cu).
#include "common.h"
#include "tma_pipeline.cuh"

namespace cb200 {

namespace {

constexpr int BM = 128, BN = 256, BK = 16;
// kATmem: the A operand of the MMAs (hi and lo) is kept in tensor memory, written there by the
// splitter warps with tcgen05.st, instead of in shared memory.  Shared-memory bandwidth is what
// bounds this kernel (TMA writes, splitter reads and writes, and the operand reads of three MMAs per
// k step all go through it); taking A out of the MMA's shared-memory reads removes a third of them.
constexpr bool kATmem = true;
constexpr int STAGES = kATmem ? 5 : 4;
constexpr int ROW_BYTES = BK * 4;                    // 64-byte rows: SWIZZLE_64B
constexpr int A_BYTES = BM * ROW_BYTES;              // 8 KB
constexpr int B_BYTES = BN * ROW_BYTES;              // 16 KB
constexpr int B_OFF = kATmem ? A_BYTES : 2 * A_BYTES;                 // raw A (+ A lo) come first in a slot
constexpr int STAGE_BYTES = B_OFF + 2 * B_BYTES;     // + raw/hi B + B lo: 40 KB (48 KB with A lo in shared)
constexpr int SPLIT_WARPS = 8;
constexpr int THREADS = (2 + SPLIT_WARPS) * 32;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;
constexpr int TMEM_A_COL = BN;                       // A ring: slot s = columns [BN + 32 s, BN + 32 s + 32): hi 16, lo 16
constexpr int TMEM_COLS = kATmem ? 512 : BN;         // accumulator: one FP32 column per column of the tile
constexpr int GROUP_M = 16;

// tcgen05 instruction descriptor, kind::tf32: D = F32, A = B = TF32, both K-major, N = 256, M = 128
constexpr uint32_t IDESC = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);

// Shared-memory matrix descriptor: K-major tile of 64-byte rows, SWIZZLE_64B, 8-row groups 512 bytes apart.
__device__ __forceinline__ uint64_t smem_desc(uint32_t saddr)
{
    uint64_t d = 0;
    d |= (uint64_t)((saddr >> 4) & 0x3fff);          // start address / 16
    d |= (uint64_t)1 << 16;                          // leading byte offset (unused for swizzled K-major)
    d |= (uint64_t)((8 * ROW_BYTES) >> 4) << 32;     // stride byte offset / 16
    d |= (uint64_t)1 << 46;                          // descriptor version of this architecture
    d |= (uint64_t)4 << 61;                          // SWIZZLE_64B
    return d;
}

__device__ __forceinline__ void umma_tf32(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t accumulate)
{
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n"
        "}\n"
        ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(IDESC), "r"(accumulate)
        : "memory");
}

// Same MMA with the A operand (128 rows = lanes, 8 k = 8 columns) read from tensor memory.
__device__ __forceinline__ void umma_tf32_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t b_desc, uint32_t accumulate)
{
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n"
        "}\n"
        ::"r"(tmem_d), "r"(tmem_a), "l"(b_desc), "r"(IDESC), "r"(accumulate)
        : "memory");
}

// 16 consecutive 32-bit columns of this thread's tensor-memory lane.
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&v)[16])
{
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),
          "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
        : "memory");
}

__device__ __forceinline__ void umma_commit(uint64_t* bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// Round to nearest TF32 (10 explicit mantissa bits), ties away from zero -- what cvt.rna.tf32.f32
// computes -- with an integer add and a mask: adding half an ulp to the magnitude carries into the
// exponent exactly when rounding must.
__device__ __forceinline__ float rn_tf32(float x)
{
    return __uint_as_float((__float_as_uint(x) + 0x1000u) & 0xffffe000u);
}

// kRewriteHi = true: hi = rn_tf32(x) is written back over the raw slab.  false: the raw FP32 slab is
// left as it is and the tensor core's own reading of an FP32 word as TF32 (it ignores the 13 low
// mantissa bits, i.e. truncates) plays the role of hi; lo is then the exact remainder of that truncation.
constexpr bool kRewriteHi = false;

__device__ __forceinline__ float trunc_tf32(float x) { return __uint_as_float(__float_as_uint(x) & 0xffffe000u); }

__device__ __forceinline__ void split4(const float4& v, float4& h, float4& l)
{
    if (!kRewriteHi) {
        l.x = rn_tf32(v.x - trunc_tf32(v.x)); l.y = rn_tf32(v.y - trunc_tf32(v.y));
        l.z = rn_tf32(v.z - trunc_tf32(v.z)); l.w = rn_tf32(v.w - trunc_tf32(v.w));
        h = v;
        return;
    }
    h.x = rn_tf32(v.x); h.y = rn_tf32(v.y); h.z = rn_tf32(v.z); h.w = rn_tf32(v.w);
    l.x = rn_tf32(v.x - h.x); l.y = rn_tf32(v.y - h.y); l.z = rn_tf32(v.z - h.z); l.w = rn_tf32(v.w - h.w);
}

// Splits the CHUNKS 16-byte chunks of a slab in place: raw -> hi, lo written lo_off bytes further.
// Four chunks per thread are in flight at a time.
template <int CHUNKS, int NTHREADS>
__device__ __forceinline__ void split_chunks(unsigned char* raw, int lo_off, int tid)
{
    static_assert(CHUNKS % NTHREADS == 0, "chunks per thread");
    constexpr int PER = CHUNKS / NTHREADS;
    float4 v[PER], h[PER], l[PER];
#pragma unroll
    for (int i = 0; i < PER; i++) v[i] = *reinterpret_cast<const float4*>(raw + (size_t)(tid + i * NTHREADS) * 16);
#pragma unroll
    for (int i = 0; i < PER; i++) split4(v[i], h[i], l[i]);
#pragma unroll
    for (int i = 0; i < PER; i++) {
        if (kRewriteHi) *reinterpret_cast<float4*>(raw + (size_t)(tid + i * NTHREADS) * 16) = h[i];
        *reinterpret_cast<float4*>(raw + lo_off + (size_t)(tid + i * NTHREADS) * 16) = l[i];
    }
}

__global__ void __launch_bounds__(THREADS, 1)
sgemm_3xtf32_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB,
                    float* __restrict__ C, size_t ldc, size_t M, size_t N, size_t K, float alpha, float beta,
                    unsigned tilesM, unsigned tilesN)
{
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* raw_full = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
    uint64_t* split_done = raw_full + STAGES;
    uint64_t* mma_done = split_done + STAGES;
    uint64_t* accum_full = mma_done + STAGES;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accum_full + 1);

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
    const int nk = (int)((K + BK - 1) / BK);
    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(&raw_full[s], 1);
            mbar_init(&split_done[s], SPLIT_WARPS);
            mbar_init(&mma_done[s], 1);
        }
        mbar_init(accum_full, 1);
        mbar_fence_init();
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------- TMA producer -------------------------------
        if (lane == 0) {
            tma_prefetch_descriptor(&mapA);
            tma_prefetch_descriptor(&mapB);
            for (int kt = 0; kt < nk; kt++) {
                const int s = kt % STAGES;
                if (kt >= STAGES && !mbar_wait(&mma_done[s], ((kt / STAGES) - 1) & 1)) break;
                unsigned char* sa = smem + s * STAGE_BYTES;
                unsigned char* sb = sa + B_OFF;
                mbar_expect_tx(&raw_full[s], A_BYTES + B_BYTES);
                tma_load_2d(sa, &mapA, kt * BK, (int)m0, &raw_full[s]);
                tma_load_2d(sb, &mapB, kt * BK, (int)n0, &raw_full[s]);
            }
        }
    } else if (warp == 1) {
        // ------------------------------- MMA issuer ---------------------------------
        if (lane == 0) {
            bool ok = true;
            for (int kt = 0; kt < nk && ok; kt++) {
                const int s = kt % STAGES;
                ok = mbar_wait(&split_done[s], (kt / STAGES) & 1);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t sa = smem_u32(smem + s * STAGE_BYTES);
                const uint32_t sb = sa + B_OFF;
                const uint64_t a_hi = smem_desc(sa), a_lo = smem_desc(sa + A_BYTES);
                const uint64_t b_hi = smem_desc(sb), b_lo = smem_desc(sb + B_BYTES);
                const uint32_t ta = tmem_base + TMEM_A_COL + s * 32;      // A hi at +0, A lo at +16
#pragma unroll
                for (int ks = 0; ks < BK / 8; ks++) {
                    const uint64_t adv = (uint64_t)((ks * 32) >> 4);      // 8 TF32 = 32 bytes along K
                    const uint32_t first = (kt > 0 || ks > 0) ? 1u : 0u;
                    if (kATmem) {
                        umma_tf32_ts(tmem_base, ta + 16 + ks * 8, b_hi + adv, first);
                        umma_tf32_ts(tmem_base, ta + ks * 8, b_lo + adv, 1u);
                        umma_tf32_ts(tmem_base, ta + ks * 8, b_hi + adv, 1u);
                    } else {
                        umma_tf32(tmem_base, a_lo + adv, b_hi + adv, first);
                        umma_tf32(tmem_base, a_hi + adv, b_lo + adv, 1u);
                        umma_tf32(tmem_base, a_hi + adv, b_hi + adv, 1u);
                    }
                }
                umma_commit(&mma_done[s]);          // slot reusable once these MMAs have read it
            }
            umma_commit(accum_full);                // accumulator complete
        }
    } else {
        // ------------------------------- splitters, then epilogue -------------------
        const int tid = threadIdx.x - 64;           // 0 .. 32*SPLIT_WARPS-1
        bool ok = true;
        for (int kt = 0; kt < nk && ok; kt++) {
            const int s = kt % STAGES;
            ok = mbar_wait(&raw_full[s], (kt / STAGES) & 1);
            if (!ok) break;
            unsigned char* sa = smem + s * STAGE_BYTES;
            unsigned char* sb = sa + B_OFF;
            if (kATmem) {
                if (warp < 6) {
                    // Warps 2-5 own the four lane quarters of tensor memory: thread = row 32q + lane of the A
                    // slab.  Its 16 k values are four 16-byte chunks; SWIZZLE_64B stored chunk j at j ^ ((row/2)&3).
                    const int row = 32 * (warp & 3) + lane;
                    uint32_t hi[16], lo[16];
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        const float4 v = *reinterpret_cast<const float4*>(sa + row * ROW_BYTES + ((j ^ ((row >> 1) & 3)) << 4));
                        float4 h, l;
                        split4(v, h, l);
                        hi[4 * j + 0] = __float_as_uint(v.x); hi[4 * j + 1] = __float_as_uint(v.y);
                        hi[4 * j + 2] = __float_as_uint(v.z); hi[4 * j + 3] = __float_as_uint(v.w);
                        lo[4 * j + 0] = __float_as_uint(l.x); lo[4 * j + 1] = __float_as_uint(l.y);
                        lo[4 * j + 2] = __float_as_uint(l.z); lo[4 * j + 3] = __float_as_uint(l.w);
                    }
                    const uint32_t taddr = tmem_base + ((uint32_t)(32 * (warp & 3)) << 16) + TMEM_A_COL + s * 32;
                    tmem_st16(taddr, hi);
                    tmem_st16(taddr + 16, lo);
                    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                }
            } else {
                split_chunks<A_BYTES / 16, SPLIT_WARPS * 32>(sa, A_BYTES, tid);
            }
            split_chunks<B_BYTES / 16, SPLIT_WARPS * 32>(sb, B_BYTES, tid);
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic writes -> visible to the MMA's async reads
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&split_done[s]);
        }
        if (ok) ok = mbar_wait(accum_full, 0);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (ok) {
            const int q = warp & 3;                 // this warp may read accumulator lanes 32q .. 32q+31
            const int half = (warp - 2) / 4;        // the two warps of a quarter take half the columns each
            const size_t row = m0 + 32 * q + lane;
            const bool useC = (beta != 0.f);
#pragma unroll 1
            for (int c = half * (BN / 64); c < (half + 1) * (BN / 64); c++) {
                uint32_t v[32];
                const uint32_t taddr = tmem_base + ((uint32_t)(32 * q) << 16) + (uint32_t)(c * 32);
                asm volatile(
                    "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                    "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                    "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                    : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
                      "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
                      "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
                      "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
                    : "r"(taddr)
                    : "memory");
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (row < M) {
#pragma unroll
                    for (int j = 0; j < 32; j++) {
                        const size_t col = n0 + c * 32 + j;
                        if (col < N) {
                            float* cc = C + row + col * ldc;
                            float r = alpha * __uint_as_float(v[j]);
                            if (useC) r = fmaf(beta, *cc, r);
                            *cc = r;
                        }
                    }
                }
            }
        }
    }

    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

}  // namespace

cudaError_t launch_sgemm_3xtf32(const GemmProblem<float>& p, cudaStream_t s)
{
    if (p.M >= (1u << 31) || p.N >= (1u << 31) || p.K >= (1u << 31)) return cudaErrorNotSupported;
    // The kernel wants A stored K x M and B stored K x N (both K-contiguous), 16-byte aligned.
    const bool fixA = !p.ta || !aligned16(p.A) || (p.lda & 3);
    const bool fixB = p.tb || !aligned16(p.B) || (p.ldb & 3);
    auto round_up = [](size_t v, size_t q) { return (v + q - 1) / q * q; };
    const size_t kld = round_up(p.K, 4);
    const size_t a_n = fixA ? kld * p.M : 0, b_n = fixB ? kld * p.N : 0;
    float* ws = nullptr;
    cudaError_t e = cudaSuccess;
    const float* A = p.A;
    const float* B = p.B;
    size_t lda = p.lda, ldb = p.ldb;
    if (fixA || fixB) {
        e = ws_alloc(reinterpret_cast<void**>(&ws), (round_up(a_n, 64) + b_n) * sizeof(float) + 256, s);
        if (e != cudaSuccess) { cudaGetLastError(); return cudaErrorNotSupported; }
        if (fixA) {
            // stored A is (ta ? K x M : M x K); transposing the M x K form gives K x M
            e = launch_repack<float>(ws, kld, p.A, p.lda, p.ta ? p.K : p.M, p.ta ? p.M : p.K, !p.ta, s);
            A = ws; lda = kld;
        }
        if (e == cudaSuccess && fixB) {
            float* wb = ws + round_up(a_n, 64);
            e = launch_repack<float>(wb, kld, p.B, p.ldb, p.tb ? p.N : p.K, p.tb ? p.K : p.N, p.tb, s);
            B = wb; ldb = kld;
        }
    }
    if (e == cudaSuccess) {
        void* enc = get_tensor_map_encoder();
        CUtensorMap mapA, mapB;
        bool ok = make_tensor_map_2d(&mapA, enc, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, A, p.K, p.M, lda, BK, BM, CU_TENSOR_MAP_SWIZZLE_64B) &&
                  make_tensor_map_2d(&mapB, enc, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, B, p.K, p.N, ldb, BK, BN, CU_TENSOR_MAP_SWIZZLE_64B);
        if (!ok) e = cudaErrorNotSupported;
        if (e == cudaSuccess) {
            static DeviceOnce once;
            e = once.run([] { return cudaFuncSetAttribute(sgemm_3xtf32_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES); });
        }
        if (e == cudaSuccess) {
            const size_t tilesM = (p.M + BM - 1) / BM, tilesN = (p.N + BN - 1) / BN;
            set_last_kernel("sgemm_3xtf32_tcgen05");
            sgemm_3xtf32_kernel<<<(unsigned)(tilesM * tilesN), THREADS, SMEM_BYTES, s>>>(
                mapA, mapB, p.C, p.ldc, p.M, p.N, p.K, p.alpha, p.beta, (unsigned)tilesM, (unsigned)tilesN);
            count_launch();
            e = cudaGetLastError();
        }
    }
    if (ws) {
        const cudaError_t e2 = ws_free(ws, s);
        if (e == cudaSuccess) e = e2;
    }
    return e;
}

unsigned sgemm_3xtf32_fault_flag() { return read_wait_timeout_flag(); }

}  // namespace cb200
