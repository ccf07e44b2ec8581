// GEMM and TRSM over the GPUs of one box, behind the C ABI.
//
// The reference's only multi-device mechanism is the queue array every entry point takes: AutoGemm
// issues its kernels round-robin over commandQueues[] (src/library/blas/xgemm.cc:603-658) and the
// solver path gives every queue one stripe of N, aligned to 128 (stripeDivision,
// src/library/blas/generic/solution_seq_make.c:764-866); all queues share the OpenCL buffers.  GPUs do
// not share buffers, so two forms exist here:
//
//  * one process (or thread) per GPU -- clblasB200{S,D}gemmSharded / {S,D}trsmSharded: every rank
//    passes its own column block of op(B) and C (GEMM) or of the right-hand sides (TRSM); the other
//    operand lives on the root and is broadcast over NCCL in column panels of the matrix as stored.
//    The broadcasts run on a second stream; the work on panel p is ordered after broadcast p only
//    (cudaEvent), so panel p+1 crosses NVLink while panel p is being used.  For GEMM with transA = N a
//    panel is a K slab and the panel products accumulate into C (beta on the first, 1 afterwards: the
//    reference's own K split, src/library/blas/specialCases/GemmSpecialCases.cpp:127-191); with
//    transA = T a panel is a block of rows of C.  For TRSM the blocked solve itself waits for the panels
//    (TrsmPanelGate): each step needs only the columns of A up to where the substitution has got.
//    The first panel is small, so little of the broadcast is exposed; later panels grow.
//  * one process, several queues -- gemm_multi_queue, reached from clblasSgemm / clblasDgemm with
//    numCommandQueues > 1: stripes of N as in the reference; a queue on another device gets copies of
//    A and of its stripes of B and C (peer copies), computes there and copies its stripe of C back.
//
// NCCL is loaded at run time (dlopen): the library carries no link-time dependency on it, and a
// process that never shards never loads it.  Remote data always lands in local memory (NCCL or a
// copy) before a kernel of this library reads it; no kernel here dereferences a peer pointer.
#include "common.h"

#include <dlfcn.h>

#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <vector>

namespace cb200 {

namespace {

// ---- the few entry points of NCCL's C ABI that are used, declared here (no nccl.h, no -lnccl) ----
typedef struct ncclComm* NcclComm;
struct NcclUniqueId { char internal[CLBLAS_B200_UNIQUE_ID_BYTES]; };
constexpr int kNcclChar = 0;            // ncclInt8 / ncclChar

struct NcclApi {
    void* handle = nullptr;
    int (*GetUniqueId)(NcclUniqueId*) = nullptr;
    int (*CommInitRank)(NcclComm*, int, NcclUniqueId, int) = nullptr;
    int (*CommInitAll)(NcclComm*, int, const int*) = nullptr;
    int (*CommDestroy)(NcclComm) = nullptr;
    int (*Broadcast)(const void*, void*, size_t, int, int, NcclComm, cudaStream_t) = nullptr;
    int (*GroupStart)() = nullptr;
    int (*GroupEnd)() = nullptr;
};

const NcclApi* nccl()
{
    static NcclApi api;
    static std::once_flag once;
    std::call_once(once, [] {
        // A copy already mapped by the process (PyTorch brings its own) is used before any other.
        void* h = nullptr;
        if (const char* path = std::getenv("CLBLAS_B200_NCCL_LIB")) h = dlopen(path, RTLD_NOW | RTLD_LOCAL);
        if (!h) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_LOCAL | RTLD_NOLOAD);
        if (!h) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_LOCAL);
        if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_LOCAL);
        if (!h) return;
        NcclApi a;
        a.handle = h;
        a.GetUniqueId = reinterpret_cast<decltype(a.GetUniqueId)>(dlsym(h, "ncclGetUniqueId"));
        a.CommInitRank = reinterpret_cast<decltype(a.CommInitRank)>(dlsym(h, "ncclCommInitRank"));
        a.CommInitAll = reinterpret_cast<decltype(a.CommInitAll)>(dlsym(h, "ncclCommInitAll"));
        a.CommDestroy = reinterpret_cast<decltype(a.CommDestroy)>(dlsym(h, "ncclCommDestroy"));
        a.Broadcast = reinterpret_cast<decltype(a.Broadcast)>(dlsym(h, "ncclBroadcast"));
        a.GroupStart = reinterpret_cast<decltype(a.GroupStart)>(dlsym(h, "ncclGroupStart"));
        a.GroupEnd = reinterpret_cast<decltype(a.GroupEnd)>(dlsym(h, "ncclGroupEnd"));
        if (a.GetUniqueId && a.CommInitRank && a.CommInitAll && a.CommDestroy && a.Broadcast && a.GroupStart && a.GroupEnd) api = a;
    });
    return api.handle ? &api : nullptr;
}

constexpr size_t kAlign = 128;          // the reference's DIVISION_ALIGNMENT, and the order of TRSM's inverted blocks

}  // namespace

// One rank's end of a communicator: the NCCL handle, the stream its collectives run on and the
// events that order that stream against the caller's.
struct ShardComm {
    NcclComm comm = nullptr;
    int nranks = 1, rank = 0, device = 0;
    cudaStream_t stream = nullptr;
    cudaEvent_t entry = nullptr;
    std::vector<cudaEvent_t> panel;
    std::mutex mu;                      // one sharded call at a time issues work through this end
};

namespace {

clblasStatus finish_comm(ShardComm* c)
{
    if (cudaGetDevice(&c->device) != cudaSuccess ||
        cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking) != cudaSuccess ||
        cudaEventCreateWithFlags(&c->entry, cudaEventDisableTiming) != cudaSuccess) {
        cudaGetLastError();
        return clblasOutOfResources;
    }
    return clblasSuccess;
}

cudaError_t panel_events(ShardComm* c, size_t n)
{
    while (c->panel.size() < n) {
        cudaEvent_t e;
        const cudaError_t err = cudaEventCreateWithFlags(&e, cudaEventDisableTiming);
        if (err != cudaSuccess) return err;
        c->panel.push_back(e);
    }
    return cudaSuccess;
}

// Column panels [b[i], b[i+1]) of a matrix with `cols` columns: a first panel of about 1/32 of the
// columns (at least min_cols), each next one four times as wide, boundaries multiples of 128, at most
// `max_panels` panels.  Every rank computes the same plan from the same arguments.  (The work on a panel
// lasts far longer than its transfer, so the panel after a small first one can already be large: few
// panels mean few short products.)
std::vector<size_t> growing_panels(size_t cols, size_t min_cols, size_t max_panels)
{
    std::vector<size_t> b{0};
    if (cols == 0) return b;
    auto up = [](size_t v) { return (v + kAlign - 1) / kAlign * kAlign; };
    size_t w = std::max(up(std::max<size_t>(min_cols, 1)), up(cols / 32));
    while (b.back() < cols) {
        size_t next = b.back() + w;
        if (next >= cols || b.size() == max_panels || cols - next < w / 2) next = cols;
        b.push_back(next);
        w *= 4;
    }
    return b;
}

// Panels of the triangular matrix of a sharded solve: a first panel of 1/32 of the columns (at least 128), each next one
// four times as wide, small panels where the substitution starts (`ascending`: at the first column).  The time the solve
// needs to reach column c grows like c^2 while the panels arrive at a constant rate, so what is exposed is the first panel
// and the waits for the next ones while the solve is still faster than the link; every broadcast costs about 45 us of its
// own.  Measured, order 8192, time per call above the rank's solve alone: this plan (256, 1024, 4096, 2816 columns) +0.55 ms
// on 2 GPUs (8192 columns per rank) and +0.66 ms on 8 (2048 per rank); equal panels of 2048 columns +0.67 / +0.83, of 512
// columns +1.22 on 2 GPUs, one broadcast of everything +0.85.
std::vector<size_t> trsm_panel_bounds(size_t n, bool ascending)
{
    std::vector<size_t> b = growing_panels(n, kAlign, 10);
    if (!ascending) {           // mirror the plan: small panels at the end of the matrix
        std::vector<size_t> m(b.size());
        for (size_t i = 0; i < b.size(); i++) {
            const size_t v = n - b[b.size() - 1 - i];
            m[i] = (i == 0) ? 0 : (i + 1 == b.size() ? n : (v + kAlign - 1) / kAlign * kAlign);
        }
        m.erase(std::unique(m.begin(), m.end()), m.end());
        b = m;
    }
    return b;
}

// Broadcast of columns [c0, c1) of a column-major matrix (rows x cols, leading dimension ld) in place:
// the memory between the first element of column c0 and the last element of column c1-1.
template <typename T>
int broadcast_columns(const NcclApi* api, ShardComm* c, T* A, size_t rows, size_t cols, size_t ld, size_t c0, size_t c1, int root)
{
    const size_t end = (c1 == cols) ? (cols - 1) * ld + rows : c1 * ld;
    const size_t first = c0 * ld;
    return api->Broadcast(A + first, A + first, (end - first) * sizeof(T), kNcclChar, root, c->comm, c->stream);
}

}  // namespace

// C <- alpha*op(A)*op(B) + beta*C on this rank's columns of op(B) and C (p: column-major problem, p.N local
// columns, p.A the broadcast operand: valid on the root, a receive buffer of the same extent elsewhere).
template <typename T>
cudaError_t gemm_sharded_colmajor(ShardComm* c, int root, const GemmProblem<T>& p, cudaStream_t s)
{
    if (c == nullptr || c->nranks <= 1) return gemm_colmajor<T>(p, s);
    const NcclApi* api = nccl();
    if (api == nullptr) return cudaErrorNotSupported;
    std::lock_guard<std::mutex> lock(c->mu);

    const size_t a_rows = p.ta ? p.K : p.M, a_cols = p.ta ? p.M : p.K;      // A as stored
    if (a_rows == 0 || a_cols == 0 || p.alpha == T(0)) return gemm_colmajor<T>(p, s);   // C <- beta*C, A not referenced: nothing travels
    // K slabs keep every tile of C in each launch, but a short K loop runs below the kernels' best rate (and the
    // large-product SGEMM kernel wants K >= 1024), so the first slab is not thinner than 1024 (float) / 512 (double);
    // row blocks of C shrink the grid of each launch, so they stay wide enough for about two waves of 128 x 128 tiles.
    size_t min_cols = sizeof(T) == 4 ? 1024 : 512;
    if (p.ta) min_cols = std::max<size_t>(kAlign, (size_t)sm_count() * 2 * 128 * 128 / std::max<size_t>(p.N, 128));
    const std::vector<size_t> b = growing_panels(a_cols, min_cols, 12);
    const size_t np = b.size() - 1;

    cudaError_t e;
    if ((e = panel_events(c, np)) != cudaSuccess) return e;
    // the broadcasts may not start before what the caller queued on `s` (producer of A on the root, last
    // reader of the receive buffer elsewhere) is done
    if ((e = cudaEventRecord(c->entry, s)) != cudaSuccess) return e;
    if ((e = cudaStreamWaitEvent(c->stream, c->entry, 0)) != cudaSuccess) return e;
    for (size_t i = 0; i < np; i++) {
        if (broadcast_columns<T>(api, c, const_cast<T*>(p.A), a_rows, a_cols, p.lda, b[i], b[i + 1], root) != 0) return cudaErrorUnknown;
        if ((e = cudaEventRecord(c->panel[i], c->stream)) != cudaSuccess) return e;
    }
    for (size_t i = 0; i < np; i++) {
        if ((e = cudaStreamWaitEvent(s, c->panel[i], 0)) != cudaSuccess) return e;
        if (p.N == 0) continue;
        GemmProblem<T> q = p;
        const size_t c0 = b[i], w = b[i + 1] - b[i];
        q.A = p.A + c0 * p.lda;
        if (!p.ta) {            // K slab: C += alpha * A[:, c0:c1] * op(B)[c0:c1, :]
            q.K = w;
            q.B = p.tb ? p.B + c0 * p.ldb : p.B + c0;
            if (i > 0) q.beta = T(1);
        } else {                // rows [c0, c1) of C
            q.M = w;
            q.C = p.C + c0;
        }
        if ((e = gemm_colmajor<T>(q, s)) != cudaSuccess) return e;
    }
    return cudaSuccess;
}

// op(A) X = alpha B (Left: this rank's columns of B) or X op(A) = alpha B (Right: this rank's rows of B);
// A valid on the root, a receive buffer elsewhere.
template <typename T>
cudaError_t trsm_sharded_colmajor(ShardComm* c, int root, bool right, bool lower, bool trans, bool unit, size_t M, size_t N,
                                  T alpha, T* A, size_t lda, T* B, size_t ldb, cudaStream_t s)
{
    if (c == nullptr || c->nranks <= 1) return trsm_colmajor<T>(right, lower, trans, unit, M, N, alpha, A, lda, B, ldb, s);
    const NcclApi* api = nccl();
    if (api == nullptr) return cudaErrorNotSupported;
    std::lock_guard<std::mutex> lock(c->mu);
    const size_t n = right ? N : M;
    if (n == 0) return cudaSuccess;
    if (alpha == T(0)) return trsm_colmajor<T>(right, lower, trans, unit, M, N, alpha, A, lda, B, ldb, s);   // A not referenced

    // The substitution starts at the first diagonal block when op(A), seen from the side it is applied on,
    // couples forwards, and at the last one otherwise; diagonal block i lives in columns [128 i, 128 (i + 1)) of
    // the stored matrix whatever the transposition.  The panels are broadcast in the order the solve reaches
    // their diagonal blocks (the off-diagonal blocks a step reads may lie in panels that come later in that
    // order -- a transposed A -- in which case that step waits for them; by then they have long arrived,
    // because the solve takes far longer than the broadcast).
    const bool ascending = ((lower != trans) != right);
    const std::vector<size_t> b = trsm_panel_bounds(n, ascending);
    const size_t np = b.size() - 1;

    cudaError_t e;
    if ((e = panel_events(c, np)) != cudaSuccess) return e;
    if ((e = cudaEventRecord(c->entry, s)) != cudaSuccess) return e;
    if ((e = cudaStreamWaitEvent(c->stream, c->entry, 0)) != cudaSuccess) return e;
    TrsmPanelGate gate;
    gate.bounds = b;
    gate.ready.resize(np);
    gate.waited.assign(np, 0);
    for (size_t k = 0; k < np; k++) {
        const size_t i = ascending ? k : np - 1 - k;
        if (broadcast_columns<T>(api, c, A, n, n, lda, b[i], b[i + 1], root) != 0) return cudaErrorUnknown;
        if ((e = cudaEventRecord(c->panel[i], c->stream)) != cudaSuccess) return e;
        gate.ready[i] = c->panel[i];
    }
    if (M != 0 && N != 0) e = trsm_colmajor<T>(right, lower, trans, unit, M, N, alpha, A, lda, B, ldb, s, &gate);
    // whatever the solve did not wait for (nothing, for a non-empty local problem) is waited for here, so that
    // the caller's stream is ordered after every broadcast of this call
    for (size_t i = 0; i < np && e == cudaSuccess; i++)
        if (!gate.waited[i]) e = cudaStreamWaitEvent(s, gate.ready[i], 0);
    return e;
}

// GEMM over several queues of one process.  Stripe q of N (boundaries multiples of 128) belongs to queue q.
// A queue on the device that holds the matrices works in place; a queue on another device receives copies.
template <typename T>
cudaError_t gemm_multi_queue(const GemmProblem<T>& p, unsigned nq, cudaStream_t* queues, cudaEvent_t* done)
{
    int home = 0;
    cudaError_t e = cudaGetDevice(&home);
    if (e != cudaSuccess) return e;
    std::vector<size_t> bounds(nq + 1);
    clblasB200PlanShards(p.N, nq, kAlign, bounds.data());
    std::vector<int> dev(nq, home);
    for (unsigned q = 0; q < nq; q++) {
        if (queues[q] == nullptr || queues[q] == cudaStreamLegacy || queues[q] == cudaStreamPerThread) continue;
        if ((e = cudaStreamGetDevice(queues[q], &dev[q])) != cudaSuccess) return e;
    }
    home = dev[0];
    constexpr size_t Q = 16 / sizeof(T);
    auto up = [](size_t v, size_t q) { return (v + q - 1) / q * q; };
    const size_t a_rows = p.ta ? p.K : p.M, a_cols = p.ta ? p.M : p.K;

    // queue 0's position at entry: the other queues may not read the operands before it
    cudaEvent_t entry = nullptr;
    if (nq > 1) {
        if ((e = cudaEventCreateWithFlags(&entry, cudaEventDisableTiming)) != cudaSuccess) return e;
        e = cudaEventRecord(entry, queues[0]);
    }
    int restore = 0;
    cudaGetDevice(&restore);
    for (unsigned q = 0; q < nq && e == cudaSuccess; q++) {
        const size_t j0 = bounds[q], nl = bounds[q + 1] - bounds[q];
        cudaStream_t s = queues[q];
        if (q > 0) e = cudaStreamWaitEvent(s, entry, 0);
        if (e != cudaSuccess) break;
        if (nl > 0) {
            GemmProblem<T> sp = p;
            sp.N = nl;
            sp.B = p.tb ? p.B + j0 : p.B + j0 * p.ldb;
            sp.C = p.C + j0 * p.ldc;
            if (dev[q] == home) {
                e = gemm_colmajor<T>(sp, s);
            } else {
                if ((e = cudaSetDevice(dev[q])) != cudaSuccess) break;
                const size_t b_rows = p.tb ? nl : p.K, b_cols = p.tb ? p.K : nl;
                const size_t lda = up(a_rows, Q), ldb = up(b_rows, Q), ldc = up(p.M, Q);
                const bool need_ab = p.K != 0 && p.alpha != T(0);
                const size_t na = need_ab ? lda * a_cols : 0, nb = need_ab ? ldb * b_cols : 0, nc = ldc * nl;
                T* ws = nullptr;
                if ((e = ws_alloc(reinterpret_cast<void**>(&ws), (up(na, 64) + up(nb, 64) + nc) * sizeof(T) + 256, s)) != cudaSuccess) break;
                T *wa = ws, *wb = ws + up(na, 64), *wc = wb + up(nb, 64);
                if (need_ab) {
                    e = cudaMemcpy2DAsync(wa, lda * sizeof(T), p.A, p.lda * sizeof(T), a_rows * sizeof(T), a_cols, cudaMemcpyDefault, s);
                    if (e == cudaSuccess)
                        e = cudaMemcpy2DAsync(wb, ldb * sizeof(T), sp.B, p.ldb * sizeof(T), b_rows * sizeof(T), b_cols, cudaMemcpyDefault, s);
                }
                if (e == cudaSuccess && p.beta != T(0))
                    e = cudaMemcpy2DAsync(wc, ldc * sizeof(T), sp.C, p.ldc * sizeof(T), p.M * sizeof(T), nl, cudaMemcpyDefault, s);
                if (e == cudaSuccess) {
                    GemmProblem<T> r = sp;
                    r.A = wa; r.lda = lda; r.B = wb; r.ldb = ldb; r.C = wc; r.ldc = ldc;
                    e = gemm_colmajor<T>(r, s);
                }
                if (e == cudaSuccess)
                    e = cudaMemcpy2DAsync(sp.C, p.ldc * sizeof(T), wc, ldc * sizeof(T), p.M * sizeof(T), nl, cudaMemcpyDefault, s);
                const cudaError_t e2 = ws_free(ws, s);
                if (e == cudaSuccess) e = e2;
            }
        }
        if (e == cudaSuccess && done != nullptr && done[q] != nullptr) e = cudaEventRecord(done[q], s);
    }
    cudaSetDevice(restore);
    if (entry) cudaEventDestroy(entry);      // released once the waits that use it have run
    return e;
}

template cudaError_t gemm_sharded_colmajor<float>(ShardComm*, int, const GemmProblem<float>&, cudaStream_t);
template cudaError_t gemm_sharded_colmajor<double>(ShardComm*, int, const GemmProblem<double>&, cudaStream_t);
template cudaError_t trsm_sharded_colmajor<float>(ShardComm*, int, bool, bool, bool, bool, size_t, size_t, float, float*, size_t,
                                                  float*, size_t, cudaStream_t);
template cudaError_t trsm_sharded_colmajor<double>(ShardComm*, int, bool, bool, bool, bool, size_t, size_t, double, double*, size_t,
                                                   double*, size_t, cudaStream_t);
template cudaError_t gemm_multi_queue<float>(const GemmProblem<float>&, unsigned, cudaStream_t*, cudaEvent_t*);
template cudaError_t gemm_multi_queue<double>(const GemmProblem<double>&, unsigned, cudaStream_t*, cudaEvent_t*);

}  // namespace cb200

using namespace cb200;

extern "C" {

clblasStatus clblasB200CommGetUniqueId(void* id)
{
    if (id == nullptr) return clblasInvalidValue;
    const NcclApi* api = nccl();
    if (api == nullptr) return clblasNotImplemented;
    NcclUniqueId u;
    if (api->GetUniqueId(&u) != 0) return clblasInvalidOperation;
    std::memcpy(id, u.internal, sizeof(u.internal));
    return clblasSuccess;
}

clblasStatus clblasB200CommInitRank(clblasB200Comm* comm, const void* id, int nranks, int rank)
{
    if (comm == nullptr || nranks < 1 || rank < 0 || rank >= nranks) return clblasInvalidValue;
    *comm = nullptr;
    ShardComm* c = new (std::nothrow) ShardComm;
    if (c == nullptr) return clblasOutOfHostMemory;
    c->nranks = nranks;
    c->rank = rank;
    if (nranks > 1) {
        const NcclApi* api = nccl();
        if (api == nullptr) { delete c; return clblasNotImplemented; }
        if (id == nullptr) { delete c; return clblasInvalidValue; }
        NcclUniqueId u;
        std::memcpy(u.internal, id, sizeof(u.internal));
        if (api->CommInitRank(&c->comm, nranks, u, rank) != 0) { delete c; return clblasInvalidOperation; }
    }
    const clblasStatus st = finish_comm(c);
    if (st != clblasSuccess) { clblasB200CommDestroy(c); return st; }
    *comm = c;
    return clblasSuccess;
}

clblasStatus clblasB200CommInitAll(clblasB200Comm* comms, int ndev, const int* devices)
{
    if (comms == nullptr || ndev < 1) return clblasInvalidValue;
    for (int i = 0; i < ndev; i++) comms[i] = nullptr;
    std::vector<NcclComm> raw(ndev, nullptr);
    if (ndev > 1) {
        const NcclApi* api = nccl();
        if (api == nullptr) return clblasNotImplemented;
        if (api->CommInitAll(raw.data(), ndev, devices) != 0) return clblasInvalidOperation;
    }
    int restore = 0;
    cudaGetDevice(&restore);
    clblasStatus st = clblasSuccess;
    for (int i = 0; i < ndev; i++) {
        ShardComm* c = new (std::nothrow) ShardComm;
        if (c == nullptr) { st = clblasOutOfHostMemory; break; }
        c->comm = raw[i];
        c->nranks = ndev;
        c->rank = i;
        comms[i] = c;
        if (cudaSetDevice(devices ? devices[i] : i) != cudaSuccess) { cudaGetLastError(); st = clblasInvalidDevice; break; }
        if ((st = finish_comm(c)) != clblasSuccess) break;
    }
    cudaSetDevice(restore);
    if (st != clblasSuccess)
        for (int i = 0; i < ndev; i++) { clblasB200CommDestroy(comms[i]); comms[i] = nullptr; }
    return st;
}

clblasStatus clblasB200CommDestroy(clblasB200Comm comm)
{
    ShardComm* c = static_cast<ShardComm*>(comm);
    if (c == nullptr) return clblasSuccess;
    int restore = 0;
    cudaGetDevice(&restore);
    cudaSetDevice(c->device);
    if (c->stream) cudaStreamSynchronize(c->stream);
    if (c->comm != nullptr) {
        const NcclApi* api = nccl();
        if (api != nullptr) api->CommDestroy(c->comm);
    }
    for (cudaEvent_t e : c->panel) cudaEventDestroy(e);
    if (c->entry) cudaEventDestroy(c->entry);
    if (c->stream) cudaStreamDestroy(c->stream);
    cudaSetDevice(restore);
    cudaGetLastError();
    delete c;
    return clblasSuccess;
}

clblasStatus clblasB200CommInfo(clblasB200Comm comm, int* nranks, int* rank)
{
    const ShardComm* c = static_cast<const ShardComm*>(comm);
    if (c == nullptr) return clblasInvalidValue;
    if (nranks) *nranks = c->nranks;
    if (rank) *rank = c->rank;
    return clblasSuccess;
}

clblasStatus clblasB200PanelPlan(size_t columns, size_t min_columns, unsigned max_panels, size_t* bounds, unsigned* count)
{
    if (bounds == nullptr || count == nullptr || max_panels == 0) return clblasInvalidValue;
    // min_columns 0 / 1: the plan of the sharded triangular solves whose substitution starts at the first / at the last
    // column (ten panels at most); otherwise that of the sharded products
    if (min_columns <= 1 && max_panels < 10) return clblasInvalidValue;
    const std::vector<size_t> b = min_columns <= 1 ? trsm_panel_bounds(columns, min_columns == 0) : growing_panels(columns, min_columns, max_panels);
    for (size_t i = 0; i < b.size(); i++) bounds[i] = b[i];
    *count = (unsigned)(b.size() - 1);
    return clblasSuccess;
}

}  // extern "C"
