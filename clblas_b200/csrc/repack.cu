// Operand repacking for GEMM: copies one operand into a 16-byte aligned, padded-ld workspace, with or
// without transposition, so that the TMA-staged kernels can take operands they cannot address in
// place (odd leading dimensions, bases offset by a few elements) and so that SGEMM always sees its
// fastest layout (A M-contiguous, B N-contiguous -- the reference's own best case, column-major
// N/T, is the one it publishes its curves on, doc/performance/clBLAS_2.6.0/S9150/README.txt:21-35).
// One pass over the operand costs (rows*cols*2*sizeof(T)) bytes of HBM traffic against
// 2*M*N*K flops of the product: below 1 % of the GEMM time once the opposite dimension exceeds
// a few thousand.  Element-granular, coalesced on both sides, any alignment; every thread keeps
// 16 independent loads in flight.
#include "common.h"

namespace cb200 {

namespace {

constexpr int COPY_COLS = 16;     // columns per CTA of the copy kernel

// dst[r + c*ldd] = src[r + c*lds], rows contiguous on both sides; CTA = 256 rows x 16 columns
template <typename T>
__global__ void __launch_bounds__(256) copy2d_kernel(T* __restrict__ dst, size_t ldd, const T* __restrict__ src, size_t lds,
                                                      size_t rows, size_t cols, unsigned tilesR)
{
    const size_t r = (size_t)(blockIdx.x % tilesR) * 256 + threadIdx.x;
    const size_t c0 = (size_t)(blockIdx.x / tilesR) * COPY_COLS;
    if (r >= rows) return;
    T v[COPY_COLS];
#pragma unroll
    for (int i = 0; i < COPY_COLS; i++) v[i] = (c0 + i < cols) ? src[r + (c0 + i) * lds] : T(0);
#pragma unroll
    for (int i = 0; i < COPY_COLS; i++)
        if (c0 + i < cols) dst[r + (c0 + i) * ldd] = v[i];
}

// dst[c + r*ldd] = src[r + c*lds]: 64 x 64 tiles through shared memory, padded against conflicts
template <typename T>
__global__ void __launch_bounds__(256) transpose2d_kernel(T* __restrict__ dst, size_t ldd, const T* __restrict__ src, size_t lds,
                                                           size_t rows, size_t cols, unsigned tilesR)
{
    __shared__ T tile[64][65];                                       // tile[c][r]
    const size_t r0 = (size_t)(blockIdx.x % tilesR) * 64, c0 = (size_t)(blockIdx.x / tilesR) * 64;
    const int tx = threadIdx.x % 64, ty = threadIdx.x / 64;          // 64 x 4
    T v[16];
#pragma unroll
    for (int i = 0; i < 16; i++) {
        const size_t r = r0 + tx, c = c0 + ty + 4 * i;
        v[i] = (r < rows && c < cols) ? src[r + c * lds] : T(0);
    }
#pragma unroll
    for (int i = 0; i < 16; i++) tile[ty + 4 * i][tx] = v[i];
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 16; i++) {
        const size_t c = c0 + tx, r = r0 + ty + 4 * i;
        if (r < rows && c < cols) dst[c + r * ldd] = tile[tx][ty + 4 * i];
    }
}

// The same transposition with 16-byte accesses on both sides, for a source whose base and leading dimension are multiples
// of 16 bytes (the destination, a workspace of this library, always is): a thread reads V = 16 / sizeof(T) consecutive
// rows of one column and later writes V consecutive columns of one row.  One 128-byte request per warp and
// instruction in the kernel above becomes four; measured on the float transposition in front of an N/N SGEMM:
// 1.46 -> about 3 TB/s.
template <typename T>
struct Vec16;
template <> struct Vec16<float> { using type = float4; };
template <> struct Vec16<double> { using type = double2; };

template <typename T>
__global__ void __launch_bounds__(256) transpose2d_vec_kernel(T* __restrict__ dst, size_t ldd, const T* __restrict__ src, size_t lds,
                                                               size_t rows, size_t cols, unsigned tilesR)
{
    constexpr int V = 16 / sizeof(T);                 // elements per 16-byte access
    constexpr int G = 64 / V;                         // threads along the vectorised direction of a 64 x 64 tile
    constexpr int P = 256 / G;                        // lines of the tile covered per pass
    using VT = typename Vec16<T>::type;
    __shared__ T tile[64][65];                                       // tile[c][r]
    const size_t r0 = (size_t)(blockIdx.x % tilesR) * 64, c0 = (size_t)(blockIdx.x / tilesR) * 64;
    const int tv = (threadIdx.x % G) * V, tl = threadIdx.x / G;
#pragma unroll
    for (int i = 0; i < 64 / P; i++) {
        const size_t r = r0 + tv, c = c0 + tl + P * i;
        T v[V];
        if (c < cols && r + V <= rows) {
            *reinterpret_cast<VT*>(v) = *reinterpret_cast<const VT*>(src + r + c * lds);
        } else {
#pragma unroll
            for (int j = 0; j < V; j++) v[j] = (c < cols && r + j < rows) ? src[r + j + c * lds] : T(0);
        }
#pragma unroll
        for (int j = 0; j < V; j++) tile[tl + P * i][tv + j] = v[j];
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 64 / P; i++) {
        const size_t c = c0 + tv, r = r0 + tl + P * i;
        if (r >= rows) continue;
        T v[V];
#pragma unroll
        for (int j = 0; j < V; j++) v[j] = tile[tv + j][tl + P * i];
        if (c + V <= cols) {
            *reinterpret_cast<VT*>(dst + c + r * ldd) = *reinterpret_cast<const VT*>(v);
        } else {
#pragma unroll
            for (int j = 0; j < V; j++)
                if (c + j < cols) dst[c + j + r * ldd] = v[j];
        }
    }
}

}  // namespace

template <typename T>
cudaError_t launch_repack(T* dst, size_t ldd, const T* src, size_t lds, size_t rows, size_t cols, bool transpose,
                          cudaStream_t s)
{
    if (rows == 0 || cols == 0) return cudaSuccess;
    if (!transpose) {
        const size_t tr = (rows + 255) / 256, tc = (cols + COPY_COLS - 1) / COPY_COLS;
        if (tr * tc >= (1ull << 31)) return cudaErrorInvalidConfiguration;
        copy2d_kernel<T><<<(unsigned)(tr * tc), 256, 0, s>>>(dst, ldd, src, lds, rows, cols, (unsigned)tr);
    } else {
        const size_t tr = (rows + 63) / 64, tc = (cols + 63) / 64;
        if (tr * tc >= (1ull << 31)) return cudaErrorInvalidConfiguration;
        constexpr size_t V = 16 / sizeof(T);
        if (aligned16(src) && aligned16(dst) && lds % V == 0 && ldd % V == 0)
            transpose2d_vec_kernel<T><<<(unsigned)(tr * tc), 256, 0, s>>>(dst, ldd, src, lds, rows, cols, (unsigned)tr);
        else
            transpose2d_kernel<T><<<(unsigned)(tr * tc), 256, 0, s>>>(dst, ldd, src, lds, rows, cols, (unsigned)tr);
    }
    count_launch();
    return cudaGetLastError();
}

template cudaError_t launch_repack<float>(float*, size_t, const float*, size_t, size_t, size_t, bool, cudaStream_t);
template cudaError_t launch_repack<double>(double*, size_t, const double*, size_t, size_t, size_t, bool, cudaStream_t);

}  // namespace cb200
