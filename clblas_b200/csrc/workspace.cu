// Library-owned device workspaces (TRSM's inverted blocks and panel, GEMM's repacked operands) come
// from one stream-ordered memory pool per device.  The pool keeps what it has been given (release
// threshold = unlimited) so that repeated calls do not go back to the driver for memory after every
// synchronisation, which is what the default pool does; clblasTeardown() destroys the pools.
// The reference allocates and releases OpenCL buffers inside each DTRSM call instead
// (src/library/blas/xtrsm.cc:1183-1207, :1499-1500).
#include "common.h"

#include <atomic>
#include <mutex>

namespace cb200 {

namespace {
std::mutex g_mu;
std::atomic<unsigned long long> g_allocs{0};
cudaMemPool_t g_pool[64] = {};

cudaError_t pool_for_current_device(cudaMemPool_t* out)
{
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> lock(g_mu);
    if (g_pool[dev] == nullptr) {
        cudaMemPoolProps props = {};
        props.allocType = cudaMemAllocationTypePinned;
        props.handleTypes = cudaMemHandleTypeNone;
        props.location.type = cudaMemLocationTypeDevice;
        props.location.id = dev;
        cudaMemPool_t pool;
        e = cudaMemPoolCreate(&pool, &props);
        if (e != cudaSuccess) return e;
        unsigned long long keep = ~0ull;
        cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &keep);
        g_pool[dev] = pool;
    }
    *out = g_pool[dev];
    return cudaSuccess;
}
}  // namespace

cudaError_t ws_alloc(void** ptr, size_t bytes, cudaStream_t s)
{
    g_allocs.fetch_add(1, std::memory_order_relaxed);
    cudaMemPool_t pool;
    cudaError_t e = pool_for_current_device(&pool);
    if (e != cudaSuccess) return e;
    return cudaMallocFromPoolAsync(ptr, bytes, pool, s);
}

unsigned long long ws_alloc_count() { return g_allocs.load(std::memory_order_relaxed); }

cudaError_t ws_free(void* ptr, cudaStream_t s) { return cudaFreeAsync(ptr, s); }

void ws_release_all()
{
    std::lock_guard<std::mutex> lock(g_mu);
    for (int d = 0; d < 64; d++) {
        if (g_pool[d] != nullptr) {
            cudaMemPoolDestroy(g_pool[d]);     // memory still in use is returned when its frees complete
            g_pool[d] = nullptr;
        }
    }
    cudaGetLastError();
}

}  // namespace cb200
