// Matrix helper API next to the level-3 routines: strided host <-> device and device <-> device copies of
// (sub-)matrices and pattern fills.
//
// Replaces clblasMatrixSizeInfo / clblasCreateMatrix* / clblas{Write,Read,Copy}{Sub,}Matrix{,Async} /
// clblasFill{Vector,SubMatrix,Matrix}{,Async} (src/clBLAS.h:9665-10238; src/library/blas/matrix.c, fill.cc).
// The reference maps them onto clEnqueue{Write,Read,Copy}BufferRect and clEnqueueFillBuffer / a 2-D fill
// kernel; here they are cudaMemcpy2DAsync on the caller's stream and one fill kernel.  Argument checks
// follow the reference: a row-major call is the column-major call with x and y exchanged, the region
// must lie inside both matrices (clblasInvalidValue otherwise), an empty region only orders the queue.
#include "common.h"

#include <algorithm>
#include <climits>
#include <cstring>

namespace cb200 {

namespace {

clblasStatus status_of(cudaError_t e)
{
    if (e == cudaSuccess) return clblasSuccess;
    cudaGetLastError();
    switch (e) {
        case cudaErrorMemoryAllocation: return clblasOutOfResources;
        case cudaErrorInvalidResourceHandle: return clblasInvalidCommandQueue;
        default: return clblasInvalidValue;
    }
}

clblasStatus begin(cudaStream_t s, unsigned nev, const clblasEvent* wait)
{
    if (nev > 0 && wait == nullptr) return clblasInvalidEventWaitList;
    for (unsigned i = 0; i < nev; i++) {
        if (wait[i] == nullptr) return clblasInvalidEventWaitList;
        if (cudaStreamWaitEvent(s, reinterpret_cast<cudaEvent_t>(wait[i]), 0) != cudaSuccess) {
            cudaGetLastError();
            return clblasInvalidEventWaitList;
        }
    }
    return clblasSuccess;
}

// Async variants record *event (created by the caller) after the work; blocking ones wait for the stream.
clblasStatus finish(cudaStream_t s, clblasEvent* event, bool blocking)
{
    if (event != nullptr && *event != nullptr) {
        const clblasStatus st = status_of(cudaEventRecord(reinterpret_cast<cudaEvent_t>(*event), s));
        if (st != clblasSuccess) return st;
    }
    if (blocking) return status_of(cudaStreamSynchronize(s));
    return clblasSuccess;
}

// inside2d of the reference (matrix.c:27-47): the w x h region at (x, y) lies inside a d1 x d2 array;
// dimensions of INT_MAX and more are refused as likely bugs.
bool inside2d(size_t d1, size_t d2, size_t x, size_t y, size_t w, size_t h)
{
    const size_t MAXDIM = (size_t)INT_MAX;
    if (d1 >= MAXDIM || d2 >= MAXDIM || w >= MAXDIM || h >= MAXDIM) return false;
    if (x >= d1 || w > d1 - x) return false;
    if (y >= d2 || h > d2 - y) return false;
    return true;
}

inline void swap_sz(size_t& a, size_t& b) { const size_t t = a; a = b; b = t; }

enum Dir { H2D, D2H, D2D };

clblasStatus copy_sub(Dir dir, clblasOrder order, size_t es, const void* A, size_t offA, size_t ldA, size_t nrA, size_t ncA,
                      size_t xA, size_t yA, void* B, size_t offB, size_t ldB, size_t nrB, size_t ncB, size_t xB, size_t yB,
                      size_t nx, size_t ny, clblasQueue q, unsigned nev, const clblasEvent* wait, clblasEvent* event,
                      bool blocking)
{
    if (order == clblasRowMajor) {
        swap_sz(xA, yA); swap_sz(nrA, ncA); swap_sz(xB, yB); swap_sz(nrB, ncB); swap_sz(nx, ny);
    }
    if (!inside2d(nrA, ncA, xA, yA, nx, ny)) return clblasInvalidValue;
    if (!inside2d(nrB, ncB, xB, yB, nx, ny)) return clblasInvalidValue;
    if (es == 0 || ldA < nrA || ldB < nrB) return clblasInvalidValue;
    if ((A == nullptr || B == nullptr) && nx != 0 && ny != 0) return clblasInvalidValue;
    cudaStream_t s = reinterpret_cast<cudaStream_t>(q);
    clblasStatus st = begin(s, nev, wait);
    if (st != clblasSuccess) return st;
    if (nx != 0 && ny != 0) {
        const char* src = static_cast<const char*>(A) + (offA + xA + yA * ldA) * es;
        char* dst = static_cast<char*>(B) + (offB + xB + yB * ldB) * es;
        const cudaMemcpyKind kind = dir == H2D ? cudaMemcpyHostToDevice : dir == D2H ? cudaMemcpyDeviceToHost : cudaMemcpyDeviceToDevice;
        st = status_of(cudaMemcpy2DAsync(dst, ldB * es, src, ldA * es, nx * es, ny, kind, s));
        if (st != clblasSuccess) return st;
    }
    return finish(s, event, blocking);
}

// Every element of an nx x ny region (column stride ld elements) receives the ES-byte pattern.
template <typename E>
__global__ void __launch_bounds__(256) fill2d_kernel(E* __restrict__ A, size_t ld, size_t nx, size_t ny, E pattern)
{
    const size_t total = nx * ny;
    for (size_t e = (size_t)blockIdx.x * 256 + threadIdx.x; e < total; e += (size_t)gridDim.x * 256)
        A[e % nx + (e / nx) * ld] = pattern;
}

// Patterns of any other size, or regions whose address is not a multiple of the element size: bytes.
__global__ void __launch_bounds__(256) fill2d_bytes_kernel(unsigned char* __restrict__ A, size_t ld_bytes, size_t nx_bytes,
                                                            size_t ny, size_t es, const unsigned char* __restrict__ pattern)
{
    const size_t total = nx_bytes * ny;
    for (size_t e = (size_t)blockIdx.x * 256 + threadIdx.x; e < total; e += (size_t)gridDim.x * 256) {
        const size_t x = e % nx_bytes;
        A[x + (e / nx_bytes) * ld_bytes] = pattern[x % es];
    }
}

template <typename E>
cudaError_t fill_typed(void* base, size_t ld, size_t nx, size_t ny, const void* pattern, cudaStream_t s)
{
    E p;
    std::memcpy(&p, pattern, sizeof(E));
    const unsigned blocks = (unsigned)std::min<size_t>((nx * ny + 255) / 256, (size_t)sm_count() * 16);
    fill2d_kernel<E><<<blocks, 256, 0, s>>>(static_cast<E*>(base), ld, nx, ny, p);
    count_launch();
    return cudaGetLastError();
}

clblasStatus fill_region(size_t es, void* A, size_t first_elem, size_t ld, size_t nx, size_t ny, const void* pattern,
                         clblasQueue q, unsigned nev, const clblasEvent* wait, clblasEvent* event, bool blocking)
{
    if (es == 0 || es > 128 || pattern == nullptr) return clblasInvalidValue;
    if (A == nullptr && nx != 0 && ny != 0) return clblasInvalidValue;
    cudaStream_t s = reinterpret_cast<cudaStream_t>(q);
    clblasStatus st = begin(s, nev, wait);
    if (st != clblasSuccess) return st;
    if (nx != 0 && ny != 0) {
        char* base = static_cast<char*>(A) + first_elem * es;
        const bool natural = (reinterpret_cast<uintptr_t>(base) % es) == 0;
        cudaError_t e;
        if (natural && es == 4) e = fill_typed<unsigned>(base, ld, nx, ny, pattern, s);
        else if (natural && es == 8) e = fill_typed<unsigned long long>(base, ld, nx, ny, pattern, s);
        else if (natural && es == 16) e = fill_typed<uint4>(base, ld, nx, ny, pattern, s);
        else if (es == 1) e = fill_typed<unsigned char>(base, ld, nx, ny, pattern, s);
        else if (natural && es == 2) e = fill_typed<unsigned short>(base, ld, nx, ny, pattern, s);
        else {
            // the pattern travels through a small stream-ordered buffer
            unsigned char* dp = nullptr;
            e = ws_alloc(reinterpret_cast<void**>(&dp), 128, s);
            if (e == cudaSuccess) {
                // pageable host memory: the bytes are staged before the call returns
                e = cudaMemcpyAsync(dp, pattern, es, cudaMemcpyHostToDevice, s);
                if (e == cudaSuccess) {
                    const unsigned blocks = (unsigned)std::min<size_t>((nx * es * ny + 255) / 256, (size_t)sm_count() * 16);
                    fill2d_bytes_kernel<<<blocks, 256, 0, s>>>(reinterpret_cast<unsigned char*>(base), ld * es, nx * es, ny, es, dp);
                    count_launch();
                    e = cudaGetLastError();
                }
                const cudaError_t e2 = ws_free(dp, s);
                if (e == cudaSuccess) e = e2;
            }
        }
        st = status_of(e);
        if (st != clblasSuccess) return st;
    }
    return finish(s, event, blocking);
}

}  // namespace

}  // namespace cb200

using namespace cb200;

extern "C" {

clblasStatus clblasMatrixSizeInfo(clblasOrder order, size_t rows, size_t columns, size_t elemsize, size_t padding,
                                  size_t* ld, size_t* fullsize)
{
    const size_t x = (order == clblasRowMajor) ? columns : rows;
    const size_t y = (order == clblasRowMajor) ? rows : columns;
    if (ld) *ld = x + padding;
    if (fullsize) *fullsize = (x + padding) * y * elemsize;
    return clblasSuccess;
}

clblasMem clblasCreateMatrix(void* context, clblasOrder order, size_t rows, size_t columns, size_t elemsize, size_t padding,
                             size_t* ld, size_t* fullsize, int* err)
{
    (void)context;
    size_t bytes = 0;
    clblasMatrixSizeInfo(order, rows, columns, elemsize, padding, ld, &bytes);
    if (fullsize) *fullsize = bytes;
    void* p = nullptr;
    const clblasStatus st = status_of(cudaMalloc(&p, bytes ? bytes : 1));
    if (err) *err = (int)st;
    return st == clblasSuccess ? p : nullptr;
}

clblasMem clblasCreateMatrixWithLd(void* context, clblasOrder order, size_t rows, size_t columns, size_t elemsize, size_t ld,
                                   size_t* fullsize, int* err)
{
    (void)context;
    const size_t inner = (order == clblasRowMajor) ? columns : rows, outer = (order == clblasRowMajor) ? rows : columns;
    if ((order != clblasRowMajor && order != clblasColumnMajor) || ld < inner) {
        if (err) *err = (int)clblasInvalidValue;
        return nullptr;
    }
    const size_t bytes = ld * outer * elemsize;
    if (fullsize) *fullsize = bytes;
    void* p = nullptr;
    const clblasStatus st = status_of(cudaMalloc(&p, bytes ? bytes : 1));
    if (err) *err = (int)st;
    return st == clblasSuccess ? p : nullptr;
}

clblasMem clblasCreateMatrixFromHost(void* context, clblasOrder order, size_t rows, size_t columns, size_t elemsize, size_t ld,
                                     void* host, size_t off_host, size_t ld_host, clblasQueue command_queue,
                                     unsigned numEventsInWaitList, const clblasEvent* eventWaitList, int* err)
{
    int e = 0;
    clblasMem m = clblasCreateMatrixWithLd(context, order, rows, columns, elemsize, ld, nullptr, &e);
    if (e == 0) {
        e = (int)clblasWriteMatrix(order, rows, columns, elemsize, host, off_host, ld_host, m, 0, ld, command_queue,
                                   numEventsInWaitList, eventWaitList);
        if (e != 0) { cudaFree(m); m = nullptr; }
    }
    if (err) *err = e;
    return m;
}

#define SUB_ARGS  A, offA, ldA, nrA, ncA, xA, yA, B, offB, ldB, nrB, ncB, xB, yB, nx, ny, command_queue, numEventsInWaitList, eventWaitList

clblasStatus clblasWriteSubMatrix(clblasOrder order, size_t element_size, const void* A, size_t offA, size_t ldA, size_t nrA,
                                  size_t ncA, size_t xA, size_t yA, clblasMem B, size_t offB, size_t ldB, size_t nrB, size_t ncB,
                                  size_t xB, size_t yB, size_t nx, size_t ny, clblasQueue command_queue,
                                  unsigned numEventsInWaitList, const clblasEvent* eventWaitList)
{
    return copy_sub(H2D, order, element_size, SUB_ARGS, nullptr, true);
}

clblasStatus clblasWriteSubMatrixAsync(clblasOrder order, size_t element_size, const void* A, size_t offA, size_t ldA, size_t nrA,
                                       size_t ncA, size_t xA, size_t yA, clblasMem B, size_t offB, size_t ldB, size_t nrB,
                                       size_t ncB, size_t xB, size_t yB, size_t nx, size_t ny, clblasQueue command_queue,
                                       unsigned numEventsInWaitList, const clblasEvent* eventWaitList, clblasEvent* event)
{
    return copy_sub(H2D, order, element_size, SUB_ARGS, event, false);
}

clblasStatus clblasReadSubMatrix(clblasOrder order, size_t element_size, const clblasMem A, size_t offA, size_t ldA, size_t nrA,
                                 size_t ncA, size_t xA, size_t yA, void* B, size_t offB, size_t ldB, size_t nrB, size_t ncB,
                                 size_t xB, size_t yB, size_t nx, size_t ny, clblasQueue command_queue,
                                 unsigned numEventsInWaitList, const clblasEvent* eventWaitList)
{
    return copy_sub(D2H, order, element_size, SUB_ARGS, nullptr, true);
}

clblasStatus clblasReadSubMatrixAsync(clblasOrder order, size_t element_size, const clblasMem A, size_t offA, size_t ldA, size_t nrA,
                                      size_t ncA, size_t xA, size_t yA, void* B, size_t offB, size_t ldB, size_t nrB, size_t ncB,
                                      size_t xB, size_t yB, size_t nx, size_t ny, clblasQueue command_queue,
                                      unsigned numEventsInWaitList, const clblasEvent* eventWaitList, clblasEvent* event)
{
    return copy_sub(D2H, order, element_size, SUB_ARGS, event, false);
}

clblasStatus clblasCopySubMatrix(clblasOrder order, size_t element_size, const clblasMem A, size_t offA, size_t ldA, size_t nrA,
                                 size_t ncA, size_t xA, size_t yA, clblasMem B, size_t offB, size_t ldB, size_t nrB, size_t ncB,
                                 size_t xB, size_t yB, size_t nx, size_t ny, clblasQueue command_queue,
                                 unsigned numEventsInWaitList, const clblasEvent* eventWaitList)
{
    return copy_sub(D2D, order, element_size, SUB_ARGS, nullptr, true);
}

clblasStatus clblasCopySubMatrixAsync(clblasOrder order, size_t element_size, const clblasMem A, size_t offA, size_t ldA, size_t nrA,
                                      size_t ncA, size_t xA, size_t yA, clblasMem B, size_t offB, size_t ldB, size_t nrB, size_t ncB,
                                      size_t xB, size_t yB, size_t nx, size_t ny, clblasQueue command_queue,
                                      unsigned numEventsInWaitList, const clblasEvent* eventWaitList, clblasEvent* event)
{
    return copy_sub(D2D, order, element_size, SUB_ARGS, event, false);
}

#undef SUB_ARGS
#define FULL_ARGS A, offA, ldA, sx, sy, 0, 0, B, offB, ldB, sx, sy, 0, 0, sx, sy, command_queue, numEventsInWaitList, eventWaitList

clblasStatus clblasWriteMatrix(clblasOrder order, size_t sx, size_t sy, size_t element_size, const void* A, size_t offA, size_t ldA,
                               clblasMem B, size_t offB, size_t ldB, clblasQueue command_queue, unsigned numEventsInWaitList,
                               const clblasEvent* eventWaitList)
{
    return copy_sub(H2D, order, element_size, FULL_ARGS, nullptr, true);
}

clblasStatus clblasWriteMatrixAsync(clblasOrder order, size_t sx, size_t sy, size_t element_size, const void* A, size_t offA,
                                    size_t ldA, clblasMem B, size_t offB, size_t ldB, clblasQueue command_queue,
                                    unsigned numEventsInWaitList, const clblasEvent* eventWaitList, clblasEvent* event)
{
    return copy_sub(H2D, order, element_size, FULL_ARGS, event, false);
}

clblasStatus clblasReadMatrix(clblasOrder order, size_t sx, size_t sy, size_t element_size, const clblasMem A, size_t offA, size_t ldA,
                              void* B, size_t offB, size_t ldB, clblasQueue command_queue, unsigned numEventsInWaitList,
                              const clblasEvent* eventWaitList)
{
    return copy_sub(D2H, order, element_size, FULL_ARGS, nullptr, true);
}

clblasStatus clblasReadMatrixAsync(clblasOrder order, size_t sx, size_t sy, size_t element_size, const clblasMem A, size_t offA,
                                   size_t ldA, void* B, size_t offB, size_t ldB, clblasQueue command_queue,
                                   unsigned numEventsInWaitList, const clblasEvent* eventWaitList, clblasEvent* event)
{
    return copy_sub(D2H, order, element_size, FULL_ARGS, event, false);
}

clblasStatus clblasCopyMatrix(clblasOrder order, size_t sx, size_t sy, size_t element_size, const clblasMem A, size_t offA, size_t ldA,
                              clblasMem B, size_t offB, size_t ldB, clblasQueue command_queue, unsigned numEventsInWaitList,
                              const clblasEvent* eventWaitList)
{
    return copy_sub(D2D, order, element_size, FULL_ARGS, nullptr, true);
}

clblasStatus clblasCopyMatrixAsync(clblasOrder order, size_t sx, size_t sy, size_t element_size, const clblasMem A, size_t offA,
                                   size_t ldA, clblasMem B, size_t offB, size_t ldB, clblasQueue command_queue,
                                   unsigned numEventsInWaitList, const clblasEvent* eventWaitList, clblasEvent* event)
{
    return copy_sub(D2D, order, element_size, FULL_ARGS, event, false);
}

#undef FULL_ARGS

clblasStatus clblasFillVectorAsync(size_t nb_elem, size_t element_size, clblasMem A, size_t offA, const void* pattern,
                                   clblasQueue command_queue, unsigned numEventsInWaitList, const clblasEvent* eventWaitList,
                                   clblasEvent* event)
{
    return fill_region(element_size, A, offA, nb_elem, nb_elem, nb_elem ? 1 : 0, pattern, command_queue, numEventsInWaitList,
                       eventWaitList, event, false);
}

clblasStatus clblasFillVector(size_t nb_elem, size_t element_size, clblasMem A, size_t offA, const void* pattern,
                              clblasQueue command_queue, unsigned numEventsInWaitList, const clblasEvent* eventWaitList)
{
    return fill_region(element_size, A, offA, nb_elem, nb_elem, nb_elem ? 1 : 0, pattern, command_queue, numEventsInWaitList,
                       eventWaitList, nullptr, true);
}

static clblasStatus fill_sub(clblasOrder order, size_t es, clblasMem A, size_t offA, size_t ldA, size_t nrA, size_t ncA, size_t xA,
                             size_t yA, size_t nx, size_t ny, const void* pattern, clblasQueue q, unsigned nev,
                             const clblasEvent* wait, clblasEvent* event, bool blocking)
{
    if (order == clblasRowMajor) { swap_sz(nrA, ncA); swap_sz(xA, yA); swap_sz(nx, ny); }
    if (!inside2d(nrA, ncA, xA, yA, nx, ny)) return clblasInvalidValue;
    if (ldA < nrA) return clblasInvalidValue;
    return fill_region(es, A, offA + xA + yA * ldA, ldA, nx, ny, pattern, q, nev, wait, event, blocking);
}

clblasStatus clblasFillSubMatrixAsync(clblasOrder order, size_t element_size, clblasMem A, size_t offA, size_t ldA, size_t nrA,
                                      size_t ncA, size_t xA, size_t yA, size_t nx, size_t ny, const void* pattern,
                                      clblasQueue command_queue, unsigned numEventsInWaitList, const clblasEvent* eventWaitList,
                                      clblasEvent* event)
{
    return fill_sub(order, element_size, A, offA, ldA, nrA, ncA, xA, yA, nx, ny, pattern, command_queue, numEventsInWaitList,
                    eventWaitList, event, false);
}

clblasStatus clblasFillSubMatrix(clblasOrder order, size_t element_size, clblasMem A, size_t offA, size_t ldA, size_t nrA,
                                 size_t ncA, size_t xA, size_t yA, size_t nx, size_t ny, const void* pattern,
                                 clblasQueue command_queue, unsigned numEventsInWaitList, const clblasEvent* eventWaitList)
{
    return fill_sub(order, element_size, A, offA, ldA, nrA, ncA, xA, yA, nx, ny, pattern, command_queue, numEventsInWaitList,
                    eventWaitList, nullptr, true);
}

clblasStatus clblasFillMatrix(clblasOrder order, size_t element_size, clblasMem A, size_t offA, size_t ldA, size_t nrA, size_t ncA,
                              const void* pattern, clblasQueue command_queue, unsigned numEventsInWaitList,
                              const clblasEvent* eventWaitList)
{
    return fill_sub(order, element_size, A, offA, ldA, nrA, ncA, 0, 0, nrA, ncA, pattern, command_queue, numEventsInWaitList,
                    eventWaitList, nullptr, true);
}

clblasStatus clblasFillMatrixAsync(clblasOrder order, size_t element_size, clblasMem A, size_t offA, size_t ldA, size_t nrA,
                                   size_t ncA, const void* pattern, clblasQueue command_queue, unsigned numEventsInWaitList,
                                   const clblasEvent* eventWaitList, clblasEvent* event)
{
    return fill_sub(order, element_size, A, offA, ldA, nrA, ncA, 0, 0, nrA, ncA, pattern, command_queue, numEventsInWaitList,
                    eventWaitList, event, false);
}

}  // extern "C"
