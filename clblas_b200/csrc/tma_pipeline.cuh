// Shared pieces of the TMA-staged GEMM kernels: mbarrier and bulk-tensor PTX wrappers, bounded
// waits, tensor-map construction on the host.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <cstdint>
#include <cstdlib>
#include <utility>

namespace cb200 {

// Set (sticky) by a kernel of the including translation unit whose bounded mbarrier wait ran out.
// One copy per translation unit; clblasB200DeviceFault() reads them all.
static __device__ unsigned int g_wait_timeout_flag;

inline unsigned read_wait_timeout_flag()
{
    unsigned v = 0;
    if (cudaMemcpyFromSymbol(&v, g_wait_timeout_flag, sizeof(v)) != cudaSuccess) { cudaGetLastError(); return 0x80000000u; }
    return v;
}

// Programmatic dependent launch.  A kernel launched through launch_pdl may start while the kernel before it on
// the stream is still running: its CTAs take SMs the earlier grid no longer needs and run their set-up (barrier
// initialisation, descriptor prefetch) there.  pdl_wait() returns once the earlier grid has completed and its
// writes are visible; every global-memory access of such a kernel comes after it.  pdl_launch_dependents() tells
// the scheduler that the next kernel may be started as far as this CTA is concerned.  Chains of short dependent
// launches (the leaves and small updates of a triangular solve) save the launch gap and the set-up time this way.
// Both instructions do nothing in a kernel that was launched the ordinary way.
//
// Off unless CLBLAS_B200_PDL=1.  Measured on B200: no gain on the solve's chains (DTRSM 8192 x 2048 27.2 with, 27.4
// TFLOP/s without; 4096 x 1024 15.7 against 16.4) and a large loss for back-to-back products whose grid is smaller than
// one wave (SGEMM N/T 1024^3: 111 us against 68 us): the CTAs of the next kernels are placed while the current one
// runs, on whatever SMs have room at that moment, so when their turn comes some SMs hold three of a kernel's CTAs and
// others none.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

inline bool pdl_enabled()
{
    static const bool on = [] { const char* v = std::getenv("CLBLAS_B200_PDL"); return v != nullptr && v[0] == '1'; }();
    return on;
}

// Only for kernels that call pdl_wait() before their first global-memory access.
template <typename... KArgs, typename... Args>
cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, Args&&... args)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

__device__ __forceinline__ uint32_t smem_u32(const void* p)
{
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}

__device__ __forceinline__ void mbar_fence_init()
{
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

// Waits for the phase with the given parity to complete.  The wait is bounded: after about two
// seconds of SM clock it records the failure in g_wait_timeout_flag and returns false, and the
// caller leaves its loop, so that a lost TMA completion can never hang the device.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity)
{
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 256; i++)
            if (mbar_try_wait(bar, parity)) return true;
        if (clock64() - t0 > 4000000000LL) {
            atomicOr(&g_wait_timeout_flag, 1u);
            return false;
        }
    }
}

// 2-D tiled bulk tensor load global -> shared, completion counted on an mbarrier.  x is the
// coordinate along the contiguous dimension; x * element size must be a multiple of 16 bytes.
// No cluster multicast is used anywhere in this library.
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y)
        : "memory");
}

__device__ __forceinline__ void tma_prefetch_descriptor(const CUtensorMap* map)
{
    asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

// Host: 2-D tensor map over a column-major matrix with `inner` contiguous elements per column,
// `outer` columns and a column stride of ld elements.  Out-of-bounds box elements read as zero.
typedef CUresult (*TensorMapEncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                           const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                           CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                           CUtensorMapFloatOOBfill);

inline bool make_tensor_map_2d(CUtensorMap* map, void* encoder, CUtensorMapDataType dt, size_t elem_bytes,
                               const void* base, size_t inner, size_t outer, size_t ld, unsigned box_inner,
                               unsigned box_outer, CUtensorMapSwizzle swizzle)
{
    if (!encoder) return false;
    cuuint64_t dims[2] = {(cuuint64_t)inner, (cuuint64_t)outer};
    cuuint64_t strides[1] = {(cuuint64_t)ld * elem_bytes};
    cuuint32_t box[2] = {box_inner, box_outer};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = reinterpret_cast<TensorMapEncodeTiledFn>(encoder)(
        map, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

}  // namespace cb200
