// Alignment-free GEMM path: C = alpha*op(A)*op(B) + beta*C for column-major operands with any
// base alignment, any leading dimension and ragged M, N, K, in ONE launch.
//
// It replaces, for operands the TMA paths cannot take, the reference's tile + row + column +
// corner launches (src/library/blas/xgemm.cc:603-658) and its unroll-1 fall-back kernels for K
// that is not a multiple of the unroll (src/library/blas/AutoGemm/KernelSelection.py:244-249):
// edges are handled by predication inside the one kernel.
//
// Structure per CTA (256 threads): element-granular, warp-coalesced global loads of the next
// K-slab into registers while the current slab is multiplied out of shared memory (two shared
// buffers, one barrier per slab); the slab is stored k-major ([k][m] and [k][n]) whatever the
// transposition, so the inner product loop reads 128-bit rows for every transpose case; each
// thread owns a TM x TN register tile split into 16-byte chunks so that a warp's shared loads
// are conflict free and its stores to C cover whole 256-byte runs of a column.
#include "common.h"

namespace cb200 {

namespace {

// 16-byte shared-memory load of V = 16/sizeof(T) consecutive elements.
__device__ __forceinline__ void lds16(const float* p, float* out)
{
    const float4 v = *reinterpret_cast<const float4*>(p);
    out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
}
__device__ __forceinline__ void lds16(const double* p, double* out)
{
    const double2 v = *reinterpret_cast<const double2*>(p);
    out[0] = v.x; out[1] = v.y;
}

template <typename T, int BM, int BN, int BK, int TM, int TN, bool TA, bool TB, bool TRI>
__global__ void __launch_bounds__((BM / TM) * (BN / TN))
gemm_simt_kernel(const GemmProblem<T> p, const unsigned tilesM)
{
    constexpr int NT = (BM / TM) * (BN / TN);
    constexpr int V = 16 / sizeof(T);          // elements per 16-byte chunk
    constexpr int LDSA = BM + V;               // padded rows: transposing stores stay conflict free
    constexpr int LDSB = BN + V;
    constexpr int CM = TM / V, CN = TN / V;    // chunks per thread along m / n
    constexpr int NTX = BM / TM;
    static_assert(NT % BM == 0 && NT % BN == 0 && NT % BK == 0, "loader mapping");
    constexpr int EA = BM * BK / NT, EB = BN * BK / NT;

    __shared__ __align__(16) T As[2][BK][LDSA];
    __shared__ __align__(16) T Bs[2][BK][LDSB];

    const int tid = threadIdx.x;
    const int tx = tid % NTX, ty = tid / NTX;
    const size_t m0 = (size_t)(blockIdx.x % tilesM) * BM;
    const size_t n0 = (size_t)(blockIdx.x / tilesM) * BN;
    const size_t M = p.M, N = p.N, K = p.K;
    if (TRI && tri_tile_outside(p.tri, m0, BM, n0, BN)) return;   // triangular update: nothing of this tile is referenced

    // ---- loader mapping: f = index along the memory-contiguous direction, s = the strided one
    constexpr int FA = TA ? BK : BM;           // extent of f for A
    constexpr int FB = TB ? BN : BK;           // op(B)(k,n): B is k-contiguous when not transposed
    const int fa = tid % FA, sa0 = tid / FA;
    const int fb = tid % FB, sb0 = tid / FB;
    constexpr int SSA = NT / FA, SSB = NT / FB;  // step of s between a thread's elements

    // A element (m,k): TA ? A[k + m*lda] : A[m + k*lda]
    const T* ga = TA ? p.A + (size_t)fa + (m0 + sa0) * p.lda : p.A + (m0 + fa) + (size_t)sa0 * p.lda;
    // B element (k,n): TB ? B[n + k*ldb] : B[k + n*ldb]
    const T* gb = TB ? p.B + (n0 + fb) + (size_t)sb0 * p.ldb : p.B + (size_t)fb + (n0 + sb0) * p.ldb;
    const size_t stepA = TA ? (size_t)BK : (size_t)BK * p.lda;   // pointer advance per K-slab
    const size_t stepB = TB ? (size_t)BK * p.ldb : (size_t)BK;
    const size_t strA = (size_t)SSA * p.lda, strB = (size_t)SSB * p.ldb;

    T ra[EA], rb[EB];
    T acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; i++)
#pragma unroll
        for (int j = 0; j < TN; j++) acc[i][j] = T(0);

    auto load_global = [&](size_t k0) {
#pragma unroll
        for (int i = 0; i < EA; i++) {
            const int s = sa0 + i * SSA;
            const bool ok = TA ? (k0 + fa < K && m0 + s < M) : (m0 + fa < M && k0 + s < K);
            ra[i] = ok ? ga[i * strA] : T(0);
        }
#pragma unroll
        for (int i = 0; i < EB; i++) {
            const int s = sb0 + i * SSB;
            const bool ok = TB ? (n0 + fb < N && k0 + s < K) : (k0 + fb < K && n0 + s < N);
            rb[i] = ok ? gb[i * strB] : T(0);
        }
        ga += stepA;
        gb += stepB;
    };
    auto store_shared = [&](int buf) {
#pragma unroll
        for (int i = 0; i < EA; i++) {
            const int s = sa0 + i * SSA;
            if (TA) As[buf][fa][s] = ra[i]; else As[buf][s][fa] = ra[i];
        }
#pragma unroll
        for (int i = 0; i < EB; i++) {
            const int s = sb0 + i * SSB;
            if (TB) Bs[buf][s][fb] = rb[i]; else Bs[buf][fb][s] = rb[i];
        }
    };

    const size_t nk = (K + BK - 1) / BK;
    if (nk > 0) {
        load_global(0);
        store_shared(0);
    }
    __syncthreads();

    for (size_t kt = 0; kt < nk; kt++) {
        const int buf = (int)(kt & 1);
        if (kt + 1 < nk) load_global((kt + 1) * BK);
#pragma unroll
        for (int k = 0; k < BK; k++) {
            T af[TM], bf[TN];
#pragma unroll
            for (int c = 0; c < CM; c++) lds16(&As[buf][k][c * (BM / CM) + tx * V], &af[c * V]);
#pragma unroll
            for (int c = 0; c < CN; c++) lds16(&Bs[buf][k][c * (BN / CN) + ty * V], &bf[c * V]);
#pragma unroll
            for (int i = 0; i < TM; i++)
#pragma unroll
                for (int j = 0; j < TN; j++) acc[i][j] = fma(af[i], bf[j], acc[i][j]);
        }
        if (kt + 1 < nk) store_shared(buf ^ 1);
        __syncthreads();
    }

    // ---- epilogue: C = alpha*acc + beta*C, beta == 0 never reads C (as the reference's B0 kernels,
    // src/library/blas/AutoGemm/KernelOpenCL.py:100-104)
    const T alpha = p.alpha, beta = p.beta;
    const bool useC = (beta != T(0));
#pragma unroll
    for (int cn = 0; cn < CN; cn++)
#pragma unroll
        for (int jn = 0; jn < V; jn++) {
            const size_t n = n0 + cn * (BN / CN) + ty * V + jn;
            if (n >= N) continue;
#pragma unroll
            for (int cm = 0; cm < CM; cm++)
#pragma unroll
                for (int jm = 0; jm < V; jm++) {
                    const size_t m = m0 + cm * (BM / CM) + tx * V + jm;
                    if (m >= M || (TRI && tri_masked(p.tri, m, n))) continue;
                    T* c = p.C + m + n * p.ldc;
                    T r = alpha * acc[cm * V + jm][cn * V + jn];
                    if (useC) r = fma(beta, *c, r);
                    *c = r;
                }
        }
}

template <typename T>
__global__ void scale_kernel(size_t M, size_t N, T beta, T* C, size_t ldc)
{
    const size_t total = M * N;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        T* c = C + (i % M) + (i / M) * ldc;
        *c = (beta == T(0)) ? T(0) : beta * *c;
    }
}

template <typename T, int BM, int BN, int BK, int TM, int TN>
cudaError_t launch_cfg(const GemmProblem<T>& p, cudaStream_t s)
{
    const size_t tilesM = (p.M + BM - 1) / BM, tilesN = (p.N + BN - 1) / BN;
    const size_t tiles = tilesM * tilesN;
    if (tiles > 0x7fffffffULL) return cudaErrorInvalidConfiguration;
    constexpr int NT = (BM / TM) * (BN / TN);
    const dim3 grid((unsigned)tiles), block(NT);
    const unsigned tm = (unsigned)tilesM;
    if (p.tri != TRI_FULL) {
        if (!p.ta && !p.tb) gemm_simt_kernel<T, BM, BN, BK, TM, TN, false, false, true><<<grid, block, 0, s>>>(p, tm);
        else if (!p.ta && p.tb) gemm_simt_kernel<T, BM, BN, BK, TM, TN, false, true, true><<<grid, block, 0, s>>>(p, tm);
        else if (p.ta && !p.tb) gemm_simt_kernel<T, BM, BN, BK, TM, TN, true, false, true><<<grid, block, 0, s>>>(p, tm);
        else gemm_simt_kernel<T, BM, BN, BK, TM, TN, true, true, true><<<grid, block, 0, s>>>(p, tm);
    } else {
        if (!p.ta && !p.tb) gemm_simt_kernel<T, BM, BN, BK, TM, TN, false, false, false><<<grid, block, 0, s>>>(p, tm);
        else if (!p.ta && p.tb) gemm_simt_kernel<T, BM, BN, BK, TM, TN, false, true, false><<<grid, block, 0, s>>>(p, tm);
        else if (p.ta && !p.tb) gemm_simt_kernel<T, BM, BN, BK, TM, TN, true, false, false><<<grid, block, 0, s>>>(p, tm);
        else gemm_simt_kernel<T, BM, BN, BK, TM, TN, true, true, false><<<grid, block, 0, s>>>(p, tm);
    }
    count_launch();
    return cudaGetLastError();
}

}  // namespace

template <typename T>
cudaError_t launch_scale(size_t M, size_t N, T beta, T* C, size_t ldc, cudaStream_t s)
{
    if (M == 0 || N == 0) return cudaSuccess;
    const size_t total = M * N;
    const unsigned blocks = (unsigned)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
    scale_kernel<T><<<blocks, 256, 0, s>>>(M, N, beta, C, ldc);
    count_launch();
    return cudaGetLastError();
}

template <>
cudaError_t launch_gemm_simt<float>(const GemmProblem<float>& p, cudaStream_t s)
{
    // Big tile once the grid fills the 148 SMs about twice; smaller tile below that so that
    // small problems still spread over the machine.
    const size_t big = ((p.M + 127) / 128) * ((p.N + 127) / 128);
    set_last_kernel("gemm_simt_ldg");
    if (big >= 2 * 148) return launch_cfg<float, 128, 128, 8, 8, 8>(p, s);
    return launch_cfg<float, 64, 64, 8, 4, 4>(p, s);
}

template <>
cudaError_t launch_gemm_simt<double>(const GemmProblem<double>& p, cudaStream_t s)
{
    set_last_kernel("gemm_simt_ldg");
    return launch_cfg<double, 64, 64, 8, 4, 4>(p, s);
}

cudaError_t gemm_simt_load_double_kernels()
{
    cudaFuncAttributes fa;
    cudaError_t e;
    if ((e = cudaFuncGetAttributes(&fa, gemm_simt_kernel<double, 64, 64, 8, 4, 4, false, false, false>)) != cudaSuccess) return e;
    if ((e = cudaFuncGetAttributes(&fa, gemm_simt_kernel<double, 64, 64, 8, 4, 4, false, true, false>)) != cudaSuccess) return e;
    if ((e = cudaFuncGetAttributes(&fa, gemm_simt_kernel<double, 64, 64, 8, 4, 4, true, false, false>)) != cudaSuccess) return e;
    if ((e = cudaFuncGetAttributes(&fa, gemm_simt_kernel<double, 64, 64, 8, 4, 4, true, true, false>)) != cudaSuccess) return e;
    return cudaFuncGetAttributes(&fa, scale_kernel<double>);
}

template cudaError_t launch_scale<float>(size_t, size_t, float, float*, size_t, cudaStream_t);
template cudaError_t launch_scale<double>(size_t, size_t, double, double*, size_t, cudaStream_t);

}  // namespace cb200
