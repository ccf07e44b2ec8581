// GEMM and TRSM on HOST matrices: clblasB200SgemmHost / clblasB200DgemmHost / clblasB200StrsmHost / clblasB200DtrsmHost.
//
// What a clBLAS program does around clblasDgemm -- clEnqueueWriteBuffer of A, B and C, the call,
// clEnqueueReadBuffer of C (src/samples/example_sgemm.c:118-160; src/client/clfunc_xgemm.hpp
// initialize_gpu_buffer / read_gpu_buffer) -- serialises PCIe and the GPU.  This entry point takes the same
// argument list with host pointers and overlaps the three: the problem is cut into column blocks of C and
// K-slabs; a copy stream uploads the pieces in the order the products need them (slab s of A and of B's
// block j, C's block j once), the compute stream multiplies block (j, s) as soon as its pieces have
// landed (beta on the first slab, 1 afterwards: the reference's split-K accumulation,
// src/library/blas/specialCases/GemmSpecialCases.cpp:127-191), and a third stream downloads block j of C
// while later blocks are still being multiplied.  Operands are laid out on the device with aligned leading
// dimensions, so every product takes the TMA kernels whatever the host leading dimensions are.
// Pinned host memory makes the copies asynchronous; pageable memory works but is staged by the driver.
// Tuning knobs (environment, read per call): CLBLAS_B200_HOST_W = width of the column blocks,
// CLBLAS_B200_HOST_NS = number of K-slabs.  On 8192^3 FP64 the defaults (2048, 4) and (2048, 2) were the best
// of eight settings; the first column block is upload-bound whatever the setting because it needs all of A.
#include "common.h"

#include <algorithm>
#include <cstdlib>
#include <mutex>
#include <vector>

namespace cb200 {

namespace {

struct HostPipe {
    std::mutex mu;
    cudaStream_t in = nullptr, cmp = nullptr, out = nullptr;
    std::vector<cudaEvent_t> events;
};
HostPipe g_pipe[64];

cudaError_t pipe_for_current_device(HostPipe** out)
{
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    HostPipe& p = g_pipe[dev];
    static std::mutex create_mu;
    std::lock_guard<std::mutex> lock(create_mu);
    if (p.in == nullptr) {
        if ((e = cudaStreamCreateWithFlags(&p.in, cudaStreamNonBlocking)) != cudaSuccess) return e;
        if ((e = cudaStreamCreateWithFlags(&p.cmp, cudaStreamNonBlocking)) != cudaSuccess) return e;
        if ((e = cudaStreamCreateWithFlags(&p.out, cudaStreamNonBlocking)) != cudaSuccess) return e;
    }
    *out = &p;
    return cudaSuccess;
}

cudaError_t event_at(HostPipe& p, size_t i, cudaEvent_t* ev)
{
    while (p.events.size() <= i) {
        cudaEvent_t e;
        cudaError_t err = cudaEventCreateWithFlags(&e, cudaEventDisableTiming);
        if (err != cudaSuccess) return err;
        p.events.push_back(e);
    }
    *ev = p.events[i];
    return cudaSuccess;
}

size_t round_up(size_t v, size_t q) { return (v + q - 1) / q * q; }

template <typename T>
cudaError_t copy2d(T* dst, size_t ldd, const T* src, size_t lds, size_t rows, size_t cols, cudaMemcpyKind kind, cudaStream_t s)
{
    if (rows == 0 || cols == 0) return cudaSuccess;
    if (ldd == rows && lds == rows) return cudaMemcpyAsync(dst, src, rows * cols * sizeof(T), kind, s);
    return cudaMemcpy2DAsync(dst, ldd * sizeof(T), src, lds * sizeof(T), rows * sizeof(T), cols, kind, s);
}

#define CK(x) do { e = (x); if (e != cudaSuccess) goto done; } while (0)

}  // namespace

// Column-major problem, host pointers already offset.  Work is ordered after what `user` holds at the time
// of the call, and `user` waits for the last download: the caller synchronises `user` (or an event recorded
// on it) before reading C.
template <typename T>
cudaError_t gemm_host_colmajor(bool ta, bool tb, size_t M, size_t N, size_t K, T alpha, const T* hA, size_t lda,
                               const T* hB, size_t ldb, T beta, T* hC, size_t ldc, cudaStream_t user)
{
    if (M == 0 || N == 0) return cudaSuccess;
    const bool product = (K != 0 && alpha != T(0));
    constexpr size_t Q = 16 / sizeof(T);
    // stored shapes (rows = contiguous direction)
    const size_t a_rows = ta ? K : M, a_cols = ta ? M : K;
    const size_t b_rows = tb ? N : K, b_cols = tb ? K : N;
    const size_t dlda = round_up(std::max<size_t>(a_rows, 1), Q), dldb = round_up(std::max<size_t>(b_rows, 1), Q), dldc = round_up(M, Q);
    const size_t a_elems = product ? dlda * a_cols : 0, b_elems = product ? dldb * b_cols : 0, c_elems = dldc * N;

    // column blocks of C: wide enough for several full waves of tiles; K-slabs: a product can start after 1/ns of A
    const size_t rows128 = (M + 127) / 128;
    size_t w = round_up(std::max<size_t>((size_t)148 * 7 / std::max<size_t>(rows128, 1), 1) * 128, 128);   // ~7 waves per product
    w = std::min(std::max<size_t>(w, 512), round_up(N, 128));
    size_t ns = !product ? 1 : K >= 8192 ? 4 : K >= 2048 ? 2 : 1;
    if (const char* v = getenv("CLBLAS_B200_HOST_W")) { const size_t x = strtoull(v, nullptr, 10); if (x) w = std::min(round_up(x, 128), round_up(N, 128)); }
    if (const char* v = getenv("CLBLAS_B200_HOST_NS")) { const size_t x = strtoull(v, nullptr, 10); if (x && product) ns = x; }
    // Block boundaries.  The first block is half as wide again as the others: its products are the ones that
    // wait for the slabs of A, so they should last as long as those uploads; what is left at the end makes a
    // narrower last block, which shortens the download that nothing overlaps.
    std::vector<size_t> bounds;
    bounds.push_back(0);
    if (N > 2 * w && getenv("CLBLAS_B200_HOST_W") == nullptr) bounds.push_back(w + w / 2);
    while (bounds.back() < N) bounds.push_back(std::min(N, bounds.back() + w));
    const size_t nb = bounds.size() - 1;
    const size_t kslab = round_up((K + ns - 1) / ns, 64);

    // One block and one slab leave nothing to overlap: everything goes on the caller's stream, without events.
    const bool single = (nb == 1 && ns == 1);
    HostPipe* pp = nullptr;
    cudaError_t e = pipe_for_current_device(&pp);
    if (e != cudaSuccess) return e;
    std::unique_lock<std::mutex> lock(pp->mu, std::defer_lock);
    if (!single) lock.lock();                     // one pipelined call per device is enqueued at a time
    HostPipe& p = *pp;
    const cudaStream_t s_in = single ? user : p.in, s_cmp = single ? user : p.cmp, s_out = single ? user : p.out;

    T* ws = nullptr;
    e = ws_alloc(reinterpret_cast<void**>(&ws), (round_up(a_elems, 64) + round_up(b_elems, 64) + c_elems) * sizeof(T) + 256, user);
    if (e != cudaSuccess) return e;
    T* dA = ws;
    T* dB = dA + round_up(a_elems, 64);
    T* dC = dB + round_up(b_elems, 64);

    cudaEvent_t ev_start, ev;
    size_t next_event = 0;
    if (!single) {
        CK(event_at(p, next_event++, &ev_start));
        CK(cudaEventRecord(ev_start, user));
        CK(cudaStreamWaitEvent(s_in, ev_start, 0));
        CK(cudaStreamWaitEvent(s_cmp, ev_start, 0));
        CK(cudaStreamWaitEvent(s_out, ev_start, 0));
    }

    for (size_t j = 0; j < nb; j++) {
        const size_t j0 = bounds[j], wj = bounds[j + 1] - j0;
        for (size_t s = 0; s < ns; s++) {
            const size_t k0 = std::min(s * kslab, K), kw = std::min(kslab, K - k0);
            if (product && kw == 0) continue;
            // ---- uploads of what product (j, s) needs and nothing has brought yet
            if (product && j == 0) {
                if (ta) CK(copy2d(dA + k0, dlda, hA + k0, lda, kw, M, cudaMemcpyHostToDevice, s_in));            // rows k0.. of the K x M matrix
                else    CK(copy2d(dA + k0 * dlda, dlda, hA + k0 * lda, lda, M, kw, cudaMemcpyHostToDevice, s_in)); // columns k0.. of M x K
            }
            if (product) {
                if (tb) CK(copy2d(dB + j0 + k0 * dldb, dldb, hB + j0 + k0 * ldb, ldb, wj, kw, cudaMemcpyHostToDevice, s_in));  // N x K stored
                else    CK(copy2d(dB + k0 + j0 * dldb, dldb, hB + k0 + j0 * ldb, ldb, kw, wj, cudaMemcpyHostToDevice, s_in));  // K x N stored
            }
            if (s == 0 && beta != T(0))
                CK(copy2d(dC + j0 * dldc, dldc, hC + j0 * ldc, ldc, M, wj, cudaMemcpyHostToDevice, s_in));
            if (!single) {
                CK(event_at(p, next_event++, &ev));
                CK(cudaEventRecord(ev, s_in));
                CK(cudaStreamWaitEvent(s_cmp, ev, 0));
            }
            // ---- the product of this block and slab
            GemmProblem<T> g;
            g.ta = ta; g.tb = tb; g.M = M; g.N = wj; g.K = product ? kw : 0;
            g.alpha = alpha; g.beta = (s == 0) ? beta : T(1);
            g.A = ta ? dA + k0 : dA + k0 * dlda; g.lda = dlda;
            g.B = tb ? dB + j0 + k0 * dldb : dB + k0 + j0 * dldb; g.ldb = dldb;
            g.C = dC + j0 * dldc; g.ldc = dldc;
            CK(gemm_colmajor<T>(g, s_cmp));
        }
        // ---- download of block j, behind its last product
        if (!single) {
            CK(event_at(p, next_event++, &ev));
            CK(cudaEventRecord(ev, s_cmp));
            CK(cudaStreamWaitEvent(s_out, ev, 0));
        }
        CK(copy2d(hC + j0 * ldc, ldc, dC + j0 * dldc, dldc, M, wj, cudaMemcpyDeviceToHost, s_out));
    }
    if (!single) {
        CK(event_at(p, next_event++, &ev));
        CK(cudaEventRecord(ev, s_out));
        CK(cudaStreamWaitEvent(user, ev, 0));
    }
    // the copy stream is done before the last product; the compute stream before the last download
done:
    if (e != cudaSuccess && !single) {
        // bring the helper streams to rest before the workspace goes back to the pool
        cudaStreamSynchronize(p.in); cudaStreamSynchronize(p.cmp); cudaStreamSynchronize(p.out);
    }
    const cudaError_t e2 = ws_free(ws, user);
    return e != cudaSuccess ? e : e2;
}

// TRSM on host matrices.  The referenced triangle of A goes up first (column panels, so that only the
// triangle crosses PCIe), then B travels in blocks of right-hand sides -- column blocks for side = Left, row
// blocks for side = Right -- which are independent systems: block j is solved while block j+1 is uploaded
// and block j-1 downloaded.
template <typename T>
cudaError_t trsm_host_colmajor(bool right, bool lower, bool trans, bool unit, size_t M, size_t N, T alpha,
                               const T* hA, size_t lda, T* hB, size_t ldb, cudaStream_t user)
{
    if (M == 0 || N == 0) return cudaSuccess;
    constexpr size_t Q = 16 / sizeof(T);
    const size_t n = right ? N : M;                    // order of A
    const size_t other = right ? M : N;                // independent right-hand sides
    const size_t dlda = round_up(n, Q), dldb = round_up(M, Q);
    const bool solve = alpha != T(0);
    const size_t nbt = std::min<size_t>(8, std::max<size_t>(1, other / 4096));
    const size_t w = round_up((other + nbt - 1) / nbt, 128);
    // Block boundaries: a first block of w/4 (the solve can start as soon as A and that little piece of B have
    // landed), full blocks of w, and a tail of two shrinking blocks (the last download overlaps nothing).
    std::vector<size_t> bounds;
    bounds.push_back(0);
    if (other > 2 * w) {
        bounds.push_back(std::max<size_t>(512, round_up(w / 4, 128)));
        while (other - bounds.back() > w + w / 2) bounds.push_back(bounds.back() + w);
        const size_t rem = other - bounds.back();
        if (rem >= 1024) bounds.push_back(bounds.back() + round_up(rem * 2 / 3, 128));
        bounds.push_back(other);
    } else {
        while (bounds.back() < other) bounds.push_back(std::min(other, bounds.back() + w));
    }
    const size_t nb = bounds.size() - 1;
    const bool single = nb == 1;

    HostPipe* pp = nullptr;
    cudaError_t e = pipe_for_current_device(&pp);
    if (e != cudaSuccess) return e;
    std::unique_lock<std::mutex> lock(pp->mu, std::defer_lock);
    if (!single) lock.lock();
    HostPipe& p = *pp;
    const cudaStream_t s_in = single ? user : p.in, s_cmp = single ? user : p.cmp, s_out = single ? user : p.out;

    const size_t a_elems = solve ? dlda * n : 0;
    T* ws = nullptr;
    e = ws_alloc(reinterpret_cast<void**>(&ws), (round_up(a_elems, 64) + dldb * N) * sizeof(T) + 256, user);
    if (e != cudaSuccess) return e;
    T* dA = ws;
    T* dB = ws + round_up(a_elems, 64);

    cudaEvent_t ev;
    size_t next_event = 0;
    if (!single) {
        CK(event_at(p, next_event++, &ev));
        CK(cudaEventRecord(ev, user));
        CK(cudaStreamWaitEvent(s_in, ev, 0));
        CK(cudaStreamWaitEvent(s_cmp, ev, 0));
        CK(cudaStreamWaitEvent(s_out, ev, 0));
    }
    if (solve) {
        // the referenced triangle, in panels of 1024 columns: rows c0.. (lower) or ..c1 (upper) of each panel
        for (size_t c0 = 0; c0 < n; c0 += 1024) {
            const size_t c1 = std::min(n, c0 + 1024);
            const size_t r0 = lower ? c0 : 0, r1 = lower ? n : c1;
            CK(copy2d(dA + r0 + c0 * dlda, dlda, hA + r0 + c0 * lda, lda, r1 - r0, c1 - c0, cudaMemcpyHostToDevice, s_in));
        }
    }
    for (size_t j = 0; j < nb; j++) {
        const size_t j0 = bounds[j], wj = bounds[j + 1] - j0;
        // block j of B: columns j0.. (Left) or rows j0.. (Right)
        T* db = right ? dB + j0 : dB + j0 * dldb;
        T* hb = right ? hB + j0 : hB + j0 * ldb;
        const size_t rows = right ? wj : M, cols = right ? N : wj;
        if (solve) CK(copy2d(db, dldb, hb, ldb, rows, cols, cudaMemcpyHostToDevice, s_in));
        if (!single) {
            CK(event_at(p, next_event++, &ev));
            CK(cudaEventRecord(ev, s_in));
            CK(cudaStreamWaitEvent(s_cmp, ev, 0));
        }
        CK(trsm_colmajor<T>(right, lower, trans, unit, rows, cols, alpha, dA, dlda, db, dldb, s_cmp));   // alpha == 0: B <- 0
        if (!single) {
            CK(event_at(p, next_event++, &ev));
            CK(cudaEventRecord(ev, s_cmp));
            CK(cudaStreamWaitEvent(s_out, ev, 0));
        }
        CK(copy2d(hb, ldb, db, dldb, rows, cols, cudaMemcpyDeviceToHost, s_out));
    }
    if (!single) {
        CK(event_at(p, next_event++, &ev));
        CK(cudaEventRecord(ev, s_out));
        CK(cudaStreamWaitEvent(user, ev, 0));
    }
done:
    if (e != cudaSuccess && !single) {
        cudaStreamSynchronize(p.in); cudaStreamSynchronize(p.cmp); cudaStreamSynchronize(p.out);
    }
    const cudaError_t e2 = ws_free(ws, user);
    return e != cudaSuccess ? e : e2;
}

#undef CK

void host_pipeline_release()
{
    for (int d = 0; d < 64; d++) {
        HostPipe& p = g_pipe[d];
        std::lock_guard<std::mutex> lock(p.mu);
        if (p.in == nullptr && p.events.empty()) continue;
        int cur = 0;
        cudaGetDevice(&cur);
        cudaSetDevice(d);
        for (cudaEvent_t ev : p.events) cudaEventDestroy(ev);
        p.events.clear();
        if (p.in) cudaStreamDestroy(p.in);
        if (p.cmp) cudaStreamDestroy(p.cmp);
        if (p.out) cudaStreamDestroy(p.out);
        p.in = p.cmp = p.out = nullptr;
        cudaSetDevice(cur);
    }
    cudaGetLastError();
}

template cudaError_t trsm_host_colmajor<float>(bool, bool, bool, bool, size_t, size_t, float, const float*, size_t, float*, size_t,
                                               cudaStream_t);
template cudaError_t trsm_host_colmajor<double>(bool, bool, bool, bool, size_t, size_t, double, const double*, size_t, double*,
                                                size_t, cudaStream_t);
template cudaError_t gemm_host_colmajor<float>(bool, bool, size_t, size_t, size_t, float, const float*, size_t, const float*, size_t,
                                               float, float*, size_t, cudaStream_t);
template cudaError_t gemm_host_colmajor<double>(bool, bool, size_t, size_t, size_t, double, const double*, size_t, const double*,
                                                size_t, double, double*, size_t, cudaStream_t);

}  // namespace cb200
