// Host front end of the C ABI declared in include/clblas_b200.h: argument checks with the
// reference's status codes and check order, row-major -> column-major normalisation, stream
// and event ordering, then the CUDA dispatchers.  No computation happens on the host.
#include "common.h"

#include <atomic>
#include <cstdlib>
#include <cstring>
#include <mutex>

namespace cb200 {

namespace {

std::atomic<unsigned long long> g_launches{0};
std::atomic<int> g_forced_path{0};
std::atomic<int> g_initialized{0};
thread_local const char* t_last_kernel = "none";
thread_local char t_last_variant[96] = "none";

// cuMemGetAddressRange through the runtime's driver entry point query: the extent of the CUDA
// allocation that holds a pointer stands in for clGetMemObjectInfo(CL_MEM_SIZE) of the
// reference's checkMatrixSizes (src/library/blas/generic/common.c:651-681).
typedef int (*MemGetAddressRangeFn)(unsigned long long*, size_t*, unsigned long long);

MemGetAddressRangeFn address_range_fn()
{
    static MemGetAddressRangeFn fn = [] {
        void* f = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &f, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            f = nullptr;
        return reinterpret_cast<MemGetAddressRangeFn>(f);
    }();
    return fn;
}

// Bytes available from `ptr` to the end of its allocation; false when the pointer is not a
// device allocation known to the driver.
bool bytes_after(const void* ptr, size_t* avail)
{
    MemGetAddressRangeFn fn = address_range_fn();
    if (!fn) return false;
    unsigned long long base = 0;
    size_t size = 0;
    if (fn(&base, &size, (unsigned long long)(uintptr_t)ptr) != 0) {
        cudaGetLastError();
        return false;
    }
    *avail = size - (size_t)((unsigned long long)(uintptr_t)ptr - base);
    return true;
}

enum ErrSet { SET_A = 0, SET_B = 1, SET_C = 2 };

clblasStatus pick(ErrSet e, clblasStatus a, clblasStatus b, clblasStatus c)
{
    return e == SET_A ? a : (e == SET_B ? b : c);
}

// checkMatrixSizes of the reference (src/library/blas/generic/common.c:585-686) for a non-packed
// rows x cols matrix op(X).
clblasStatus check_matrix_sizes(size_t tsize, clblasOrder order, clblasTranspose trans, size_t rows, size_t cols,
                                const void* buf, size_t off, size_t ld, ErrSet e)
{
    if (rows == 0 || cols == 0) return clblasInvalidDim;
    const bool tra = (order == clblasRowMajor && trans != clblasNoTrans) ||
                     (order == clblasColumnMajor && trans == clblasNoTrans);
    size_t matr;
    if (tra) {
        if (ld < rows) return pick(e, clblasInvalidLeadDimA, clblasInvalidLeadDimB, clblasInvalidLeadDimC);
        matr = ((cols - 1) * ld + rows) * tsize;
    } else {
        if (ld < cols) return pick(e, clblasInvalidLeadDimA, clblasInvalidLeadDimB, clblasInvalidLeadDimC);
        matr = ((rows - 1) * ld + cols) * tsize;
    }
    size_t avail = 0;
    if (!bytes_after(buf, &avail)) return pick(e, clblasInvalidMatA, clblasInvalidMatB, clblasInvalidMatC);
    const size_t offb = off * tsize;
    if (offb + matr > avail || offb + matr < offb)
        return pick(e, clblasInsufficientMemMatA, clblasInsufficientMemMatB, clblasInsufficientMemMatC);
    return clblasSuccess;
}

// checkQueues / checkEventWaitList (src/library/blas/functor/include/functor_utils.h:22-60).  A
// NULL cudaStream_t inside the array is the legacy default stream and therefore legal here.
clblasStatus check_queues(unsigned n, clblasQueue* q)
{
    if (n == 0 || q == nullptr) return clblasInvalidCommandQueue;
    return clblasSuccess;
}

clblasStatus check_events(unsigned n, const clblasEvent* ev)
{
    if (n > 0 && ev == nullptr) return clblasInvalidEventWaitList;
    for (unsigned i = 0; i < n; i++)
        if (ev[i] == nullptr) return clblasInvalidEventWaitList;
    return clblasSuccess;
}

clblasStatus from_cuda(cudaError_t e)
{
    switch (e) {
        case cudaSuccess: return clblasSuccess;
        case cudaErrorMemoryAllocation: return clblasOutOfResources;
        case cudaErrorInvalidValue: return clblasInvalidValue;
        case cudaErrorInvalidResourceHandle: return clblasInvalidCommandQueue;
        case cudaErrorNotSupported: return clblasNotImplemented;
        default: return clblasInvalidOperation;
    }
}

clblasStatus wait_all(cudaStream_t s, unsigned n, const clblasEvent* ev)
{
    for (unsigned i = 0; i < n; i++) {
        cudaError_t e = cudaStreamWaitEvent(s, reinterpret_cast<cudaEvent_t>(ev[i]), 0);
        if (e != cudaSuccess) { cudaGetLastError(); return clblasInvalidEventWaitList; }
    }
    return clblasSuccess;
}

// Completion events.  events[0] is recorded on the queue that did the work; a caller that passed several
// queues gets events[q] recorded on queue q once the work is done (the reference hands out one event per
// queue, src/library/blas/xgemm.cc:606-610, src/library/blas/generic/solution_seq_make.c:402-404).
clblasStatus record_out(unsigned nq, clblasQueue* queues, clblasEvent* events)
{
    if (events == nullptr) return clblasSuccess;
    cudaStream_t s0 = reinterpret_cast<cudaStream_t>(queues[0]);
    cudaEvent_t done = reinterpret_cast<cudaEvent_t>(events[0]);
    if (done != nullptr && cudaEventRecord(done, s0) != cudaSuccess) { cudaGetLastError(); return clblasInvalidValue; }
    bool others = false;
    for (unsigned q = 1; q < nq; q++) others = others || events[q] != nullptr;
    if (!others) return clblasSuccess;
    cudaEvent_t tmp = nullptr;
    if (done == nullptr) {
        if (cudaEventCreateWithFlags(&tmp, cudaEventDisableTiming) != cudaSuccess || cudaEventRecord(tmp, s0) != cudaSuccess) {
            cudaGetLastError();
            return clblasOutOfResources;
        }
        done = tmp;
    }
    clblasStatus st = clblasSuccess;
    for (unsigned q = 1; q < nq && st == clblasSuccess; q++) {
        if (events[q] == nullptr) continue;
        cudaStream_t sq = reinterpret_cast<cudaStream_t>(queues[q]);
        if (cudaStreamWaitEvent(sq, done, 0) != cudaSuccess || cudaEventRecord(reinterpret_cast<cudaEvent_t>(events[q]), sq) != cudaSuccess) {
            cudaGetLastError();
            st = clblasInvalidValue;
        }
    }
    if (tmp) cudaEventDestroy(tmp);
    return st;
}

// Column-major form of a GEMM call.  Row-major C (M x N) is column-major C^T (N x M) = op(B)^T * op(A)^T: the
// operands, their transposition flags and M with N are exchanged (the reference's force_gemm_column_major,
// src/library/blas/xgemm.cc:40-61).  ConjTrans means Trans for real types.
template <typename T>
GemmProblem<T> normalise_gemm(clblasOrder order, clblasTranspose transA, clblasTranspose transB, size_t M, size_t N, size_t K,
                              T alpha, const void* A, size_t offA, size_t lda, const void* B, size_t offB, size_t ldb,
                              T beta, void* C, size_t offC, size_t ldc)
{
    GemmProblem<T> p;
    p.alpha = alpha; p.beta = beta; p.K = K;
    p.C = static_cast<T*>(C) + offC; p.ldc = ldc;
    const bool ta = transA != clblasNoTrans, tb = transB != clblasNoTrans;
    if (order == clblasColumnMajor) {
        p.ta = ta; p.tb = tb; p.M = M; p.N = N;
        p.A = static_cast<const T*>(A) + offA; p.lda = lda;
        p.B = static_cast<const T*>(B) + offB; p.ldb = ldb;
    } else {
        p.ta = tb; p.tb = ta; p.M = N; p.N = M;
        p.A = static_cast<const T*>(B) + offB; p.lda = ldb;
        p.B = static_cast<const T*>(A) + offA; p.ldb = lda;
    }
    return p;
}

template <typename T>
clblasStatus gemm_entry(clblasOrder order, clblasTranspose transA, clblasTranspose transB,
                        size_t M, size_t N, size_t K, T alpha,
                        const void* A, size_t offA, size_t lda, const void* B, size_t offB, size_t ldb,
                        T beta, void* C, size_t offC, size_t ldc,
                        unsigned nq, clblasQueue* queues, unsigned nev, const clblasEvent* wait, clblasEvent* events)
{
    // xgemm.cc:685-706: memory objects first, then (K != 0) A and B sizes, then C sizes.
    if (A == nullptr) return clblasInvalidMatA;
    if (B == nullptr) return clblasInvalidMatB;
    if (C == nullptr) return clblasInvalidMatC;
    if (order != clblasRowMajor && order != clblasColumnMajor) return clblasInvalidValue;
    if ((unsigned)transA > 2u || (unsigned)transB > 2u) return clblasInvalidValue;
    clblasStatus st;
    if (K != 0) {
        if ((st = check_matrix_sizes(sizeof(T), order, transA, M, K, A, offA, lda, SET_A)) != clblasSuccess) return st;
        if ((st = check_matrix_sizes(sizeof(T), order, transB, K, N, B, offB, ldb, SET_B)) != clblasSuccess) return st;
    }
    if ((st = check_matrix_sizes(sizeof(T), order, clblasNoTrans, M, N, C, offC, ldc, SET_C)) != clblasSuccess) return st;
    if ((st = check_queues(nq, queues)) != clblasSuccess) return st;
    if ((st = check_events(nev, wait)) != clblasSuccess) return st;

    cudaStream_t s = reinterpret_cast<cudaStream_t>(queues[0]);
    for (unsigned q = 0; q < nq; q++)
        if ((st = wait_all(reinterpret_cast<cudaStream_t>(queues[q]), nev, wait)) != clblasSuccess) return st;

    const GemmProblem<T> p = normalise_gemm<T>(order, transA, transB, M, N, K, alpha, A, offA, lda, B, offB, ldb, beta, C, offC, ldc);
    if (nq > 1) {
        // Several queues: stripes of N, one per queue, as the reference's multi-queue GEMM does.
        cudaError_t e = gemm_multi_queue<T>(p, nq, reinterpret_cast<cudaStream_t*>(queues), reinterpret_cast<cudaEvent_t*>(events));
        if (e != cudaSuccess) { cudaGetLastError(); return from_cuda(e); }
        return clblasSuccess;
    }
    cudaError_t e = gemm_colmajor<T>(p, s);
    if (e != cudaSuccess) { cudaGetLastError(); return from_cuda(e); }
    return record_out(nq, queues, events);
}

// The GEMM front end on one rank's shard (clblasB200{S,D}gemmSharded): the checks of gemm_entry, except that a
// rank may own no columns at all (its part of the split is empty) and still takes part in the broadcasts.
template <typename T>
clblasStatus gemm_sharded_entry(clblasOrder order, clblasTranspose transA, clblasTranspose transB,
                                size_t M, size_t N, size_t K, T alpha,
                                void* A, size_t offA, size_t lda, void* B, size_t offB, size_t ldb,
                                T beta, void* C, size_t offC, size_t ldc, clblasB200Comm comm, int root,
                                unsigned nq, clblasQueue* queues, unsigned nev, const clblasEvent* wait, clblasEvent* events)
{
    if (A == nullptr) return clblasInvalidMatA;
    if (B == nullptr) return clblasInvalidMatB;
    if (C == nullptr) return clblasInvalidMatC;
    if (order != clblasRowMajor && order != clblasColumnMajor) return clblasInvalidValue;
    if ((unsigned)transA > 2u || (unsigned)transB > 2u) return clblasInvalidValue;
    int nranks = 1, rank = 0;
    if (comm != nullptr) clblasB200CommInfo(comm, &nranks, &rank);
    if (root < 0 || root >= nranks) return clblasInvalidValue;
    // The sharded dimension is N for a column-major call and M for a row-major one (the columns of the
    // column-major view of C either way); the operand that is broadcast is the other one's partner: A for
    // column-major, B for row-major.
    const bool col = order == clblasColumnMajor;
    const size_t local = col ? N : M;
    clblasStatus st;
    if (K != 0) {
        if (col || local != 0)
            if ((st = check_matrix_sizes(sizeof(T), order, transA, M, K, A, offA, lda, SET_A)) != clblasSuccess) return st;
        if (!col || local != 0)
            if ((st = check_matrix_sizes(sizeof(T), order, transB, K, N, B, offB, ldb, SET_B)) != clblasSuccess) return st;
    }
    if (local != 0 && (st = check_matrix_sizes(sizeof(T), order, clblasNoTrans, M, N, C, offC, ldc, SET_C)) != clblasSuccess) return st;
    if ((st = check_queues(nq, queues)) != clblasSuccess) return st;
    if ((st = check_events(nev, wait)) != clblasSuccess) return st;
    cudaStream_t s = reinterpret_cast<cudaStream_t>(queues[0]);
    if ((st = wait_all(s, nev, wait)) != clblasSuccess) return st;
    const GemmProblem<T> p = normalise_gemm<T>(order, transA, transB, M, N, K, alpha, A, offA, lda, B, offB, ldb, beta, C, offC, ldc);
    cudaError_t e = gemm_sharded_colmajor<T>(static_cast<ShardComm*>(comm), root, p, s);
    if (e != cudaSuccess) { cudaGetLastError(); return from_cuda(e); }
    return record_out(nq, queues, events);
}

// The TRSM front end on one rank's shard (clblasB200{S,D}trsmSharded): checks of trsm_entry; the dimension of B
// that is not the order of A is the sharded one and may be zero on a rank.
template <typename T>
clblasStatus trsm_sharded_entry(clblasOrder order, clblasSide side, clblasUplo uplo, clblasTranspose transA, clblasDiag diag,
                                size_t M, size_t N, T alpha, void* A, size_t offA, size_t lda, void* B, size_t offB, size_t ldb,
                                clblasB200Comm comm, int root,
                                unsigned nq, clblasQueue* queues, unsigned nev, const clblasEvent* wait, clblasEvent* events)
{
    clblasStatus st;
    if ((st = check_queues(nq, queues)) != clblasSuccess) return st;
    if ((st = check_events(nev, wait)) != clblasSuccess) return st;
    if (!g_initialized.load()) return clblasNotInitialized;
    if (A == nullptr) return clblasInvalidMatA;
    if (B == nullptr) return clblasInvalidMatB;
    if (order != clblasRowMajor && order != clblasColumnMajor) return clblasInvalidValue;
    if ((unsigned)side > 1u || (unsigned)uplo > 1u || (unsigned)transA > 2u || (unsigned)diag > 1u) return clblasInvalidValue;
    int nranks = 1, rank = 0;
    if (comm != nullptr) clblasB200CommInfo(comm, &nranks, &rank);
    if (root < 0 || root >= nranks) return clblasInvalidValue;
    const size_t msize = (side == clblasLeft) ? M : N, other = (side == clblasLeft) ? N : M;
    if ((st = check_matrix_sizes(sizeof(T), order, transA, msize, msize, A, offA, lda, SET_A)) != clblasSuccess) return st;
    if (other != 0 && (st = check_matrix_sizes(sizeof(T), order, clblasNoTrans, M, N, B, offB, ldb, SET_B)) != clblasSuccess) return st;

    cudaStream_t s = reinterpret_cast<cudaStream_t>(queues[0]);
    if ((st = wait_all(s, nev, wait)) != clblasSuccess) return st;
    bool right = (side == clblasRight), lower = (uplo == clblasLower);
    if (order == clblasRowMajor) {
        size_t t = M; M = N; N = t;
        right = !right;
        lower = !lower;
    }
    cudaError_t e = trsm_sharded_colmajor<T>(static_cast<ShardComm*>(comm), root, right, lower, transA != clblasNoTrans,
                                             diag == clblasUnit, M, N, alpha, static_cast<T*>(A) + offA, lda,
                                             static_cast<T*>(B) + offB, ldb, s);
    if (e != cudaSuccess) { cudaGetLastError(); return from_cuda(e); }
    return record_out(nq, queues, events);
}

// Complex GEMM front end: the checks of gemm_entry on complex elements (2 * sizeof(R) bytes each).
template <typename R>
clblasStatus cgemm_entry(clblasOrder order, clblasTranspose transA, clblasTranspose transB,
                         size_t M, size_t N, size_t K, R ar, R ai,
                         const void* A, size_t offA, size_t lda, const void* B, size_t offB, size_t ldb,
                         R br, R bi, void* C, size_t offC, size_t ldc,
                         unsigned nq, clblasQueue* queues, unsigned nev, const clblasEvent* wait, clblasEvent* events)
{
    if (A == nullptr) return clblasInvalidMatA;
    if (B == nullptr) return clblasInvalidMatB;
    if (C == nullptr) return clblasInvalidMatC;
    if (order != clblasRowMajor && order != clblasColumnMajor) return clblasInvalidValue;
    if ((unsigned)transA > 2u || (unsigned)transB > 2u) return clblasInvalidValue;
    clblasStatus st;
    const size_t tsize = 2 * sizeof(R);
    if (K != 0) {
        if ((st = check_matrix_sizes(tsize, order, transA, M, K, A, offA, lda, SET_A)) != clblasSuccess) return st;
        if ((st = check_matrix_sizes(tsize, order, transB, K, N, B, offB, ldb, SET_B)) != clblasSuccess) return st;
    }
    if ((st = check_matrix_sizes(tsize, order, clblasNoTrans, M, N, C, offC, ldc, SET_C)) != clblasSuccess) return st;
    if ((st = check_queues(nq, queues)) != clblasSuccess) return st;
    if ((st = check_events(nev, wait)) != clblasSuccess) return st;

    cudaStream_t s = reinterpret_cast<cudaStream_t>(queues[0]);
    if ((st = wait_all(s, nev, wait)) != clblasSuccess) return st;

    const R* a = static_cast<const R*>(A) + 2 * offA;
    const R* b = static_cast<const R*>(B) + 2 * offB;
    R* c = static_cast<R*>(C) + 2 * offC;
    cudaError_t e;
    if (order == clblasColumnMajor)
        e = cgemm_colmajor<R>((int)transA, (int)transB, M, N, K, ar, ai, a, lda, b, ldb, br, bi, c, ldc, s);
    else    // row-major C is column-major C^T = op(B)^T * op(A)^T; a conjugation stays with its operand
        e = cgemm_colmajor<R>((int)transB, (int)transA, N, M, K, ar, ai, b, ldb, a, lda, br, bi, c, ldc, s);
    if (e != cudaSuccess) { cudaGetLastError(); return from_cuda(e); }
    return record_out(nq, queues, events);
}

// Leading-dimension check of checkMatrixSizes for a matrix in host memory (no allocation extent to compare with).
clblasStatus check_host_matrix(clblasOrder order, clblasTranspose trans, size_t rows, size_t cols, size_t ld, ErrSet e)
{
    if (rows == 0 || cols == 0) return clblasInvalidDim;
    const bool tra = (order == clblasRowMajor && trans != clblasNoTrans) || (order == clblasColumnMajor && trans == clblasNoTrans);
    if (ld < (tra ? rows : cols)) return pick(e, clblasInvalidLeadDimA, clblasInvalidLeadDimB, clblasInvalidLeadDimC);
    return clblasSuccess;
}

// GEMM on host matrices: the checks of gemm_entry in the same order, then the pipelined upload / multiply / download.
template <typename T>
clblasStatus gemm_host_entry(clblasOrder order, clblasTranspose transA, clblasTranspose transB,
                             size_t M, size_t N, size_t K, T alpha,
                             const void* A, size_t offA, size_t lda, const void* B, size_t offB, size_t ldb,
                             T beta, void* C, size_t offC, size_t ldc,
                             unsigned nq, clblasQueue* queues, unsigned nev, const clblasEvent* wait, clblasEvent* events)
{
    if (A == nullptr) return clblasInvalidMatA;
    if (B == nullptr) return clblasInvalidMatB;
    if (C == nullptr) return clblasInvalidMatC;
    if (order != clblasRowMajor && order != clblasColumnMajor) return clblasInvalidValue;
    if ((unsigned)transA > 2u || (unsigned)transB > 2u) return clblasInvalidValue;
    clblasStatus st;
    if (K != 0) {
        if ((st = check_host_matrix(order, transA, M, K, lda, SET_A)) != clblasSuccess) return st;
        if ((st = check_host_matrix(order, transB, K, N, ldb, SET_B)) != clblasSuccess) return st;
    }
    if ((st = check_host_matrix(order, clblasNoTrans, M, N, ldc, SET_C)) != clblasSuccess) return st;
    if ((st = check_queues(nq, queues)) != clblasSuccess) return st;
    if ((st = check_events(nev, wait)) != clblasSuccess) return st;

    cudaStream_t s = reinterpret_cast<cudaStream_t>(queues[0]);
    if ((st = wait_all(s, nev, wait)) != clblasSuccess) return st;
    const T* a = static_cast<const T*>(A) + offA;
    const T* b = static_cast<const T*>(B) + offB;
    T* c = static_cast<T*>(C) + offC;
    const bool ta = transA != clblasNoTrans, tb = transB != clblasNoTrans;
    cudaError_t e;
    if (order == clblasColumnMajor) e = gemm_host_colmajor<T>(ta, tb, M, N, K, alpha, a, lda, b, ldb, beta, c, ldc, s);
    else                            e = gemm_host_colmajor<T>(tb, ta, N, M, K, alpha, b, ldb, a, lda, beta, c, ldc, s);
    if (e != cudaSuccess) { cudaGetLastError(); return from_cuda(e); }
    return record_out(nq, queues, events);
}

// TRSM on host matrices: the checks of trsm_entry in the same order (without memory extents).
template <typename T>
clblasStatus trsm_host_entry(clblasOrder order, clblasSide side, clblasUplo uplo, clblasTranspose transA, clblasDiag diag,
                             size_t M, size_t N, T alpha, const void* A, size_t offA, size_t lda, void* B, size_t offB, size_t ldb,
                             unsigned nq, clblasQueue* queues, unsigned nev, const clblasEvent* wait, clblasEvent* events)
{
    clblasStatus st;
    if ((st = check_queues(nq, queues)) != clblasSuccess) return st;
    if ((st = check_events(nev, wait)) != clblasSuccess) return st;
    if (!g_initialized.load()) return clblasNotInitialized;
    if (A == nullptr) return clblasInvalidMatA;
    if (B == nullptr) return clblasInvalidMatB;
    if (order != clblasRowMajor && order != clblasColumnMajor) return clblasInvalidValue;
    if ((unsigned)side > 1u || (unsigned)uplo > 1u || (unsigned)transA > 2u || (unsigned)diag > 1u) return clblasInvalidValue;
    const size_t msize = (side == clblasLeft) ? M : N;
    if ((st = check_host_matrix(order, transA, msize, msize, lda, SET_A)) != clblasSuccess) return st;
    if ((st = check_host_matrix(order, clblasNoTrans, M, N, ldb, SET_B)) != clblasSuccess) return st;

    cudaStream_t s = reinterpret_cast<cudaStream_t>(queues[0]);
    if ((st = wait_all(s, nev, wait)) != clblasSuccess) return st;
    bool right = (side == clblasRight), lower = (uplo == clblasLower);
    if (order == clblasRowMajor) {
        size_t t = M; M = N; N = t;
        right = !right;
        lower = !lower;
    }
    cudaError_t e = trsm_host_colmajor<T>(right, lower, transA != clblasNoTrans, diag == clblasUnit, M, N, alpha,
                                          static_cast<const T*>(A) + offA, lda, static_cast<T*>(B) + offB, ldb, s);
    if (e != cudaSuccess) { cudaGetLastError(); return from_cuda(e); }
    return record_out(nq, queues, events);
}

// Complex SYRK / HERK, SYR2K / HER2K, SYMM / HEMM front ends.  Checks in the order of the reference's doSyrk /
// doHerk (src/library/blas/xsyrk.c:48-70, xherk.c:52-85), doSyr2k / doHer2k and doSymm (xsymm.c, shared by HEMM).
// A symmetric update refuses clblasConjTrans and a Hermitian one clblasTrans (clblasInvalidValue), as there.
// Row-major calls become column-major calls on the transposed problem: other triangle, other transposition
// (N <-> T, or N <-> C with alpha conjugated for the Hermitian rank-2k update), other side for SYMM / HEMM.
template <typename R>
clblasStatus csyrk_entry(bool herm, bool two, clblasOrder order, clblasUplo uplo, clblasTranspose trans, size_t N, size_t K,
                         R ar, R ai, const void* A, size_t offA, size_t lda, const void* B, size_t offB, size_t ldb,
                         R br, R bi, void* C, size_t offC, size_t ldc,
                         unsigned nq, clblasQueue* queues, unsigned nev, const clblasEvent* wait, clblasEvent* events)
{
    clblasStatus st;
    if (!g_initialized.load()) return clblasNotInitialized;
    if (nq == 0 || queues == nullptr) return clblasInvalidValue;
    if (nev != 0 && wait == nullptr) return clblasInvalidEventWaitList;
    if (A == nullptr) return clblasInvalidMatA;
    if (two && B == nullptr) return clblasInvalidMatB;
    if (C == nullptr) return clblasInvalidMatC;
    if (order != clblasRowMajor && order != clblasColumnMajor) return clblasInvalidValue;
    if ((unsigned)uplo > 1u || (unsigned)trans > 2u) return clblasInvalidValue;
    if (trans == (herm ? clblasTrans : clblasConjTrans)) return clblasInvalidValue;
    const size_t tsize = 2 * sizeof(R);
    if ((st = check_matrix_sizes(tsize, order, trans, N, K, A, offA, lda, SET_A)) != clblasSuccess) return st;
    if (two && (st = check_matrix_sizes(tsize, order, trans, N, K, B, offB, ldb, SET_B)) != clblasSuccess) return st;
    if ((st = check_matrix_sizes(tsize, order, clblasNoTrans, N, N, C, offC, ldc, SET_C)) != clblasSuccess) return st;
    if ((st = check_events(nev, wait)) != clblasSuccess) return st;

    cudaStream_t s = reinterpret_cast<cudaStream_t>(queues[0]);
    if ((st = wait_all(s, nev, wait)) != clblasSuccess) return st;
    bool lower = (uplo == clblasLower);
    int op = (trans == clblasNoTrans) ? 0 : (herm ? 2 : 1);
    if (order == clblasRowMajor) {
        lower = !lower;
        op = (op == 0) ? (herm ? 2 : 1) : 0;
        if (herm && two) ai = -ai;
    }
    const R* a = static_cast<const R*>(A) + 2 * offA;
    R* c = static_cast<R*>(C) + 2 * offC;
    cudaError_t e;
    if (two) e = csyr2k_colmajor<R>(herm, lower, op, N, K, ar, ai, a, lda, static_cast<const R*>(B) + 2 * offB, ldb, br, bi, c, ldc, s);
    else     e = csyrk_colmajor<R>(herm, lower, op, N, K, ar, ai, a, lda, br, bi, c, ldc, s);
    if (e != cudaSuccess) { cudaGetLastError(); return from_cuda(e); }
    return record_out(nq, queues, events);
}

template <typename R>
clblasStatus csymm_entry(bool herm, clblasOrder order, clblasSide side, clblasUplo uplo, size_t M, size_t N, R ar, R ai,
                         const void* A, size_t offA, size_t lda, const void* B, size_t offB, size_t ldb, R br, R bi,
                         void* C, size_t offC, size_t ldc,
                         unsigned nq, clblasQueue* queues, unsigned nev, const clblasEvent* wait, clblasEvent* events)
{
    clblasStatus st;
    if (!g_initialized.load()) return clblasNotInitialized;
    if (A == nullptr) return clblasInvalidMatA;
    if (B == nullptr) return clblasInvalidMatB;
    if (C == nullptr) return clblasInvalidMatC;
    if (order != clblasRowMajor && order != clblasColumnMajor) return clblasInvalidValue;
    if ((unsigned)side > 1u || (unsigned)uplo > 1u) return clblasInvalidValue;
    const size_t n = (side == clblasLeft) ? M : N;
    const size_t tsize = 2 * sizeof(R);
    if ((st = check_matrix_sizes(tsize, order, clblasNoTrans, n, n, A, offA, lda, SET_A)) != clblasSuccess) return st;
    if ((st = check_matrix_sizes(tsize, order, clblasNoTrans, M, N, B, offB, ldb, SET_B)) != clblasSuccess) return st;
    if ((st = check_matrix_sizes(tsize, order, clblasNoTrans, M, N, C, offC, ldc, SET_C)) != clblasSuccess) return st;
    if (nq == 0 || queues == nullptr) return clblasInvalidValue;
    if (nev != 0 && wait == nullptr) return clblasInvalidEventWaitList;

    cudaStream_t s = reinterpret_cast<cudaStream_t>(queues[0]);
    if ((st = wait_all(s, nev, wait)) != clblasSuccess) return st;
    bool right = (side == clblasRight), lower = (uplo == clblasLower);
    if (order == clblasRowMajor) {
        size_t t = M; M = N; N = t;
        right = !right;
        lower = !lower;
    }
    cudaError_t e = csymm_colmajor<R>(herm, right, lower, M, N, ar, ai, static_cast<const R*>(A) + 2 * offA, lda,
                                      static_cast<const R*>(B) + 2 * offB, ldb, br, bi, static_cast<R*>(C) + 2 * offC, ldc, s);
    if (e != cudaSuccess) { cudaGetLastError(); return from_cuda(e); }
    return record_out(nq, queues, events);
}

// Complex TRMM front end: the checks of trmm_entry on complex elements.
template <typename R>
clblasStatus ctrmm_entry(clblasOrder order, clblasSide side, clblasUplo uplo, clblasTranspose transA, clblasDiag diag,
                         size_t M, size_t N, R ar, R ai, const void* A, size_t offA, size_t lda,
                         void* B, size_t offB, size_t ldb,
                         unsigned nq, clblasQueue* queues, unsigned nev, const clblasEvent* wait, clblasEvent* events)
{
    clblasStatus st;
    if (!g_initialized.load()) return clblasNotInitialized;
    if (A == nullptr) return clblasInvalidMatA;
    if (B == nullptr) return clblasInvalidMatB;
    if (order != clblasRowMajor && order != clblasColumnMajor) return clblasInvalidValue;
    if ((unsigned)side > 1u || (unsigned)uplo > 1u || (unsigned)transA > 2u || (unsigned)diag > 1u) return clblasInvalidValue;
    const size_t msize = (side == clblasLeft) ? M : N;
    const size_t tsize = 2 * sizeof(R);
    if ((st = check_matrix_sizes(tsize, order, transA, msize, msize, A, offA, lda, SET_A)) != clblasSuccess) return st;
    if ((st = check_matrix_sizes(tsize, order, clblasNoTrans, M, N, B, offB, ldb, SET_B)) != clblasSuccess) return st;
    if ((st = check_queues(nq, queues)) != clblasSuccess) return st;
    if ((st = check_events(nev, wait)) != clblasSuccess) return st;

    cudaStream_t s = reinterpret_cast<cudaStream_t>(queues[0]);
    if ((st = wait_all(s, nev, wait)) != clblasSuccess) return st;
    bool right = (side == clblasRight), lower = (uplo == clblasLower);
    if (order == clblasRowMajor) {
        size_t t = M; M = N; N = t;
        right = !right;
        lower = !lower;
    }
    cudaError_t e = ctrmm_colmajor<R>(right, lower, (int)transA, diag == clblasUnit, M, N, ar, ai,
                                      static_cast<const R*>(A) + 2 * offA, lda, static_cast<R*>(B) + 2 * offB, ldb, s);
    if (e != cudaSuccess) { cudaGetLastError(); return from_cuda(e); }
    return record_out(nq, queues, events);
}

template <typename T>
clblasStatus trsm_entry(clblasOrder order, clblasSide side, clblasUplo uplo, clblasTranspose transA, clblasDiag diag,
                        size_t M, size_t N, T alpha, const void* A, size_t offA, size_t lda,
                        void* B, size_t offB, size_t ldb,
                        unsigned nq, clblasQueue* queues, unsigned nev, const clblasEvent* wait, clblasEvent* events)
{
    // xtrsm.cc:1623-1624 then functor_xtrsm.cc:57-75.
    clblasStatus st;
    if ((st = check_queues(nq, queues)) != clblasSuccess) return st;
    if ((st = check_events(nev, wait)) != clblasSuccess) return st;
    if (!g_initialized.load()) return clblasNotInitialized;
    if (A == nullptr) return clblasInvalidMatA;
    if (B == nullptr) return clblasInvalidMatB;
    if (order != clblasRowMajor && order != clblasColumnMajor) return clblasInvalidValue;
    if ((unsigned)side > 1u || (unsigned)uplo > 1u || (unsigned)transA > 2u || (unsigned)diag > 1u) return clblasInvalidValue;
    const size_t msize = (side == clblasLeft) ? M : N;
    if ((st = check_matrix_sizes(sizeof(T), order, transA, msize, msize, A, offA, lda, SET_A)) != clblasSuccess) return st;
    if ((st = check_matrix_sizes(sizeof(T), order, clblasNoTrans, M, N, B, offB, ldb, SET_B)) != clblasSuccess) return st;

    cudaStream_t s = reinterpret_cast<cudaStream_t>(queues[0]);
    if ((st = wait_all(s, nev, wait)) != clblasSuccess) return st;

    bool right = (side == clblasRight), lower = (uplo == clblasLower);
    if (order == clblasRowMajor) {
        // A row-major matrix is its transpose in column-major: B^T gets solved from the other side
        // with the other triangle (the reference's force_trsm_column_major, xtrsm.cc:54-64).
        size_t t = M; M = N; N = t;
        right = !right;
        lower = !lower;
    }
    cudaError_t e = trsm_colmajor<T>(right, lower, transA != clblasNoTrans, diag == clblasUnit, M, N, alpha,
                                     static_cast<const T*>(A) + offA, lda, static_cast<T*>(B) + offB, ldb, s);
    if (e != cudaSuccess) { cudaGetLastError(); return from_cuda(e); }
    return record_out(nq, queues, events);
}

// clblasStrmm / clblasDtrmm: checks of the reference's doTrmm (src/library/blas/xtrmm.c:52-70):
// initialised, memory objects, A (order x order), B; then the same row-major flip as TRSM.
// Complex TRSM front end: the checks of trsm_entry on complex elements.
template <typename R>
clblasStatus ctrsm_entry(clblasOrder order, clblasSide side, clblasUplo uplo, clblasTranspose transA, clblasDiag diag,
                         size_t M, size_t N, R ar, R ai, const void* A, size_t offA, size_t lda,
                         void* B, size_t offB, size_t ldb,
                         unsigned nq, clblasQueue* queues, unsigned nev, const clblasEvent* wait, clblasEvent* events)
{
    clblasStatus st;
    if ((st = check_queues(nq, queues)) != clblasSuccess) return st;
    if ((st = check_events(nev, wait)) != clblasSuccess) return st;
    if (!g_initialized.load()) return clblasNotInitialized;
    if (A == nullptr) return clblasInvalidMatA;
    if (B == nullptr) return clblasInvalidMatB;
    if (order != clblasRowMajor && order != clblasColumnMajor) return clblasInvalidValue;
    if ((unsigned)side > 1u || (unsigned)uplo > 1u || (unsigned)transA > 2u || (unsigned)diag > 1u) return clblasInvalidValue;
    const size_t msize = (side == clblasLeft) ? M : N;
    const size_t tsize = 2 * sizeof(R);
    if ((st = check_matrix_sizes(tsize, order, transA, msize, msize, A, offA, lda, SET_A)) != clblasSuccess) return st;
    if ((st = check_matrix_sizes(tsize, order, clblasNoTrans, M, N, B, offB, ldb, SET_B)) != clblasSuccess) return st;

    cudaStream_t s = reinterpret_cast<cudaStream_t>(queues[0]);
    if ((st = wait_all(s, nev, wait)) != clblasSuccess) return st;
    bool right = (side == clblasRight), lower = (uplo == clblasLower);
    if (order == clblasRowMajor) {
        // a row-major matrix is its transpose in column-major: the other side, the other triangle, M and N exchanged
        size_t t = M; M = N; N = t;
        right = !right;
        lower = !lower;
    }
    cudaError_t e = ctrsm_colmajor<R>(right, lower, (int)transA, diag == clblasUnit, M, N, ar, ai,
                                      static_cast<const R*>(A) + 2 * offA, lda, static_cast<R*>(B) + 2 * offB, ldb, s);
    if (e != cudaSuccess) { cudaGetLastError(); return from_cuda(e); }
    return record_out(nq, queues, events);
}

template <typename T>
clblasStatus trmm_entry(clblasOrder order, clblasSide side, clblasUplo uplo, clblasTranspose transA, clblasDiag diag,
                        size_t M, size_t N, T alpha, const void* A, size_t offA, size_t lda,
                        void* B, size_t offB, size_t ldb,
                        unsigned nq, clblasQueue* queues, unsigned nev, const clblasEvent* wait, clblasEvent* events)
{
    clblasStatus st;
    if (!g_initialized.load()) return clblasNotInitialized;
    if (A == nullptr) return clblasInvalidMatA;
    if (B == nullptr) return clblasInvalidMatB;
    if (order != clblasRowMajor && order != clblasColumnMajor) return clblasInvalidValue;
    if ((unsigned)side > 1u || (unsigned)uplo > 1u || (unsigned)transA > 2u || (unsigned)diag > 1u) return clblasInvalidValue;
    const size_t msize = (side == clblasLeft) ? M : N;
    if ((st = check_matrix_sizes(sizeof(T), order, transA, msize, msize, A, offA, lda, SET_A)) != clblasSuccess) return st;
    if ((st = check_matrix_sizes(sizeof(T), order, clblasNoTrans, M, N, B, offB, ldb, SET_B)) != clblasSuccess) return st;
    if ((st = check_queues(nq, queues)) != clblasSuccess) return st;
    if ((st = check_events(nev, wait)) != clblasSuccess) return st;

    cudaStream_t s = reinterpret_cast<cudaStream_t>(queues[0]);
    if ((st = wait_all(s, nev, wait)) != clblasSuccess) return st;
    bool right = (side == clblasRight), lower = (uplo == clblasLower);
    if (order == clblasRowMajor) {
        size_t t = M; M = N; N = t;
        right = !right;
        lower = !lower;
    }
    cudaError_t e = trmm_colmajor<T>(right, lower, transA != clblasNoTrans, diag == clblasUnit, M, N, alpha,
                                     static_cast<const T*>(A) + offA, lda, static_cast<T*>(B) + offB, ldb, s);
    if (e != cudaSuccess) { cudaGetLastError(); return from_cuda(e); }
    return record_out(nq, queues, events);
}

// clblasSsyrk / clblasDsyrk: checks of the reference's doSyrk (src/library/blas/xsyrk.c:48-70): initialised,
// queues (InvalidValue there), memory objects A and C, A sizes (N x K as op(A)), C sizes (N x N).
template <typename T>
clblasStatus syrk_entry(clblasOrder order, clblasUplo uplo, clblasTranspose transA, size_t N, size_t K, T alpha,
                        const void* A, size_t offA, size_t lda, T beta, void* C, size_t offC, size_t ldc,
                        unsigned nq, clblasQueue* queues, unsigned nev, const clblasEvent* wait, clblasEvent* events)
{
    clblasStatus st;
    if (!g_initialized.load()) return clblasNotInitialized;
    if (nq == 0 || queues == nullptr) return clblasInvalidValue;
    if (A == nullptr) return clblasInvalidMatA;
    if (C == nullptr) return clblasInvalidMatC;
    if (order != clblasRowMajor && order != clblasColumnMajor) return clblasInvalidValue;
    if ((unsigned)uplo > 1u || (unsigned)transA > 2u) return clblasInvalidValue;
    if ((st = check_matrix_sizes(sizeof(T), order, transA, N, K, A, offA, lda, SET_A)) != clblasSuccess) return st;
    if ((st = check_matrix_sizes(sizeof(T), order, clblasNoTrans, N, N, C, offC, ldc, SET_C)) != clblasSuccess) return st;
    if ((st = check_events(nev, wait)) != clblasSuccess) return st;

    cudaStream_t s = reinterpret_cast<cudaStream_t>(queues[0]);
    if ((st = wait_all(s, nev, wait)) != clblasSuccess) return st;
    bool lower = (uplo == clblasLower), trans = (transA != clblasNoTrans);
    if (order == clblasRowMajor) {
        // a row-major matrix is its transpose in column-major: the other triangle of C, and A^T stored
        lower = !lower;
        trans = !trans;
    }
    cudaError_t e = syrk_colmajor<T>(lower, trans, N, K, alpha, static_cast<const T*>(A) + offA, lda, beta,
                                     static_cast<T*>(C) + offC, ldc, s);
    if (e != cudaSuccess) { cudaGetLastError(); return from_cuda(e); }
    return record_out(nq, queues, events);
}

// SYR2K front end.  Check order of the reference's doSyr2k (src/library/blas/xsyr2k.c:52-78).
template <typename T>
clblasStatus syr2k_entry(clblasOrder order, clblasUplo uplo, clblasTranspose transAB, size_t N, size_t K, T alpha,
                         const void* A, size_t offA, size_t lda, const void* B, size_t offB, size_t ldb, T beta,
                         void* C, size_t offC, size_t ldc,
                         unsigned nq, clblasQueue* queues, unsigned nev, const clblasEvent* wait, clblasEvent* events)
{
    clblasStatus st;
    if (!g_initialized.load()) return clblasNotInitialized;
    if (nq == 0 || queues == nullptr) return clblasInvalidValue;
    if (A == nullptr) return clblasInvalidMatA;
    if (B == nullptr) return clblasInvalidMatB;
    if (C == nullptr) return clblasInvalidMatC;
    if (order != clblasRowMajor && order != clblasColumnMajor) return clblasInvalidValue;
    if ((unsigned)uplo > 1u || (unsigned)transAB > 2u) return clblasInvalidValue;
    if ((st = check_matrix_sizes(sizeof(T), order, transAB, N, K, A, offA, lda, SET_A)) != clblasSuccess) return st;
    if ((st = check_matrix_sizes(sizeof(T), order, transAB, N, K, B, offB, ldb, SET_B)) != clblasSuccess) return st;
    if ((st = check_matrix_sizes(sizeof(T), order, clblasNoTrans, N, N, C, offC, ldc, SET_C)) != clblasSuccess) return st;
    if ((st = check_events(nev, wait)) != clblasSuccess) return st;

    cudaStream_t s = reinterpret_cast<cudaStream_t>(queues[0]);
    if ((st = wait_all(s, nev, wait)) != clblasSuccess) return st;
    bool lower = (uplo == clblasLower), trans = (transAB != clblasNoTrans);
    if (order == clblasRowMajor) {
        lower = !lower;
        trans = !trans;
    }
    cudaError_t e = syr2k_colmajor<T>(lower, trans, N, K, alpha, static_cast<const T*>(A) + offA, lda,
                                      static_cast<const T*>(B) + offB, ldb, beta, static_cast<T*>(C) + offC, ldc, s);
    if (e != cudaSuccess) { cudaGetLastError(); return from_cuda(e); }
    return record_out(nq, queues, events);
}

// SYMM front end.  Check order of the reference's doSymm (src/library/blas/xsymm.c): memory objects and
// sizes first, then the queues and the wait list; a row-major call is the column-major call on the
// transposed problem (other side, other triangle, M and N exchanged), as there.
template <typename T>
clblasStatus symm_entry(clblasOrder order, clblasSide side, clblasUplo uplo, size_t M, size_t N, T alpha,
                        const void* A, size_t offA, size_t lda, const void* B, size_t offB, size_t ldb, T beta,
                        void* C, size_t offC, size_t ldc,
                        unsigned nq, clblasQueue* queues, unsigned nev, const clblasEvent* wait, clblasEvent* events)
{
    clblasStatus st;
    if (!g_initialized.load()) return clblasNotInitialized;
    if (A == nullptr) return clblasInvalidMatA;
    if (B == nullptr) return clblasInvalidMatB;
    if (C == nullptr) return clblasInvalidMatC;
    if (order != clblasRowMajor && order != clblasColumnMajor) return clblasInvalidValue;
    if ((unsigned)side > 1u || (unsigned)uplo > 1u) return clblasInvalidValue;
    const size_t n = (side == clblasLeft) ? M : N;
    if ((st = check_matrix_sizes(sizeof(T), order, clblasNoTrans, n, n, A, offA, lda, SET_A)) != clblasSuccess) return st;
    if ((st = check_matrix_sizes(sizeof(T), order, clblasNoTrans, M, N, B, offB, ldb, SET_B)) != clblasSuccess) return st;
    if ((st = check_matrix_sizes(sizeof(T), order, clblasNoTrans, M, N, C, offC, ldc, SET_C)) != clblasSuccess) return st;
    if (nq == 0 || queues == nullptr) return clblasInvalidValue;
    if (nev != 0 && wait == nullptr) return clblasInvalidEventWaitList;

    cudaStream_t s = reinterpret_cast<cudaStream_t>(queues[0]);
    if ((st = wait_all(s, nev, wait)) != clblasSuccess) return st;
    bool right = (side == clblasRight), lower = (uplo == clblasLower);
    if (order == clblasRowMajor) {
        size_t t = M; M = N; N = t;
        right = !right;
        lower = !lower;
    }
    cudaError_t e = symm_colmajor<T>(right, lower, M, N, alpha, static_cast<const T*>(A) + offA, lda,
                                     static_cast<const T*>(B) + offB, ldb, beta, static_cast<T*>(C) + offC, ldc, s);
    if (e != cudaSuccess) { cudaGetLastError(); return from_cuda(e); }
    return record_out(nq, queues, events);
}

}  // namespace

void count_launch(unsigned n) { g_launches.fetch_add(n, std::memory_order_relaxed); }
void set_last_kernel(const char* name) { t_last_kernel = name; set_last_variant(name); }
void set_last_variant(const char* name)
{
    std::strncpy(t_last_variant, name, sizeof(t_last_variant) - 1);
    t_last_variant[sizeof(t_last_variant) - 1] = 0;
}
int forced_gemm_path() { return g_forced_path.load(std::memory_order_relaxed); }

int sm_count()
{
    static std::atomic<int> cached[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    int v = cached[dev].load(std::memory_order_relaxed);
    if (v == 0) {
        if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) v = 148;
        cached[dev].store(v, std::memory_order_relaxed);
    }
    return v;
}

void* get_tensor_map_encoder()
{
    static void* fn = [] {
        void* f = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            f = nullptr;
        return f;
    }();
    return fn;
}

}  // namespace cb200

using namespace cb200;

extern "C" {

clblasStatus clblasGetVersion(unsigned* major, unsigned* minor, unsigned* patch)
{
    if (!major || !minor || !patch) return clblasInvalidValue;
    *major = 2; *minor = 12; *patch = 0;
    return clblasSuccess;
}

clblasStatus clblasSetup(void)
{
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || n == 0) { cudaGetLastError(); return clblasInvalidDevice; }
    // Implementation switch by environment variable, in the manner of the reference's
    // AMD_CLBLAS_GEMM_IMPLEMENTATION (src/library/blas/impl.c:81-129):
    // CLBLAS_B200_GEMM_PATH = 0 (automatic), 1 (alignment-free kernels), 4 (SGEMM: 3xTF32 on tcgen05).
    if (const char* env = std::getenv("CLBLAS_B200_GEMM_PATH")) {
        const int v = std::atoi(env);
        if (v >= 0 && v <= 4) g_forced_path.store(v);
    }
    g_initialized.store(1);
    return clblasSuccess;
}

void clblasTeardown(void)
{
    host_pipeline_release();
    trsm_release_workspaces();
    g_initialized.store(0);
}

clblasStatus clblasSgemm(clblasOrder order, clblasTranspose transA, clblasTranspose transB, size_t M, size_t N, size_t K,
                         float alpha, const clblasMem A, size_t offA, size_t lda, const clblasMem B, size_t offB, size_t ldb,
                         float beta, clblasMem C, size_t offC, size_t ldc, unsigned nq, clblasQueue* queues,
                         unsigned nev, const clblasEvent* wait, clblasEvent* events)
{
    return gemm_entry<float>(order, transA, transB, M, N, K, alpha, A, offA, lda, B, offB, ldb, beta, C, offC, ldc,
                             nq, queues, nev, wait, events);
}

clblasStatus clblasDgemm(clblasOrder order, clblasTranspose transA, clblasTranspose transB, size_t M, size_t N, size_t K,
                         double alpha, const clblasMem A, size_t offA, size_t lda, const clblasMem B, size_t offB, size_t ldb,
                         double beta, clblasMem C, size_t offC, size_t ldc, unsigned nq, clblasQueue* queues,
                         unsigned nev, const clblasEvent* wait, clblasEvent* events)
{
    return gemm_entry<double>(order, transA, transB, M, N, K, alpha, A, offA, lda, B, offB, ldb, beta, C, offC, ldc,
                              nq, queues, nev, wait, events);
}

clblasStatus clblasStrsm(clblasOrder order, clblasSide side, clblasUplo uplo, clblasTranspose transA, clblasDiag diag,
                         size_t M, size_t N, float alpha, const clblasMem A, size_t offA, size_t lda,
                         clblasMem B, size_t offB, size_t ldb, unsigned nq, clblasQueue* queues,
                         unsigned nev, const clblasEvent* wait, clblasEvent* events)
{
    return trsm_entry<float>(order, side, uplo, transA, diag, M, N, alpha, A, offA, lda, B, offB, ldb,
                             nq, queues, nev, wait, events);
}

clblasStatus clblasDtrsm(clblasOrder order, clblasSide side, clblasUplo uplo, clblasTranspose transA, clblasDiag diag,
                         size_t M, size_t N, double alpha, const clblasMem A, size_t offA, size_t lda,
                         clblasMem B, size_t offB, size_t ldb, unsigned nq, clblasQueue* queues,
                         unsigned nev, const clblasEvent* wait, clblasEvent* events)
{
    return trsm_entry<double>(order, side, uplo, transA, diag, M, N, alpha, A, offA, lda, B, offB, ldb,
                              nq, queues, nev, wait, events);
}

clblasStatus clblasStrmm(clblasOrder order, clblasSide side, clblasUplo uplo, clblasTranspose transA, clblasDiag diag,
                         size_t M, size_t N, float alpha, const clblasMem A, size_t offA, size_t lda,
                         clblasMem B, size_t offB, size_t ldb, unsigned nq, clblasQueue* queues,
                         unsigned nev, const clblasEvent* wait, clblasEvent* events)
{
    return trmm_entry<float>(order, side, uplo, transA, diag, M, N, alpha, A, offA, lda, B, offB, ldb,
                             nq, queues, nev, wait, events);
}

clblasStatus clblasDtrmm(clblasOrder order, clblasSide side, clblasUplo uplo, clblasTranspose transA, clblasDiag diag,
                         size_t M, size_t N, double alpha, const clblasMem A, size_t offA, size_t lda,
                         clblasMem B, size_t offB, size_t ldb, unsigned nq, clblasQueue* queues,
                         unsigned nev, const clblasEvent* wait, clblasEvent* events)
{
    return trmm_entry<double>(order, side, uplo, transA, diag, M, N, alpha, A, offA, lda, B, offB, ldb,
                              nq, queues, nev, wait, events);
}

clblasStatus clblasSsyrk(clblasOrder order, clblasUplo uplo, clblasTranspose transA, size_t N, size_t K, float alpha,
                         const clblasMem A, size_t offA, size_t lda, float beta, clblasMem C, size_t offC, size_t ldc,
                         unsigned nq, clblasQueue* queues, unsigned nev, const clblasEvent* wait, clblasEvent* events)
{
    return syrk_entry<float>(order, uplo, transA, N, K, alpha, A, offA, lda, beta, C, offC, ldc, nq, queues, nev, wait, events);
}

clblasStatus clblasDsyrk(clblasOrder order, clblasUplo uplo, clblasTranspose transA, size_t N, size_t K, double alpha,
                         const clblasMem A, size_t offA, size_t lda, double beta, clblasMem C, size_t offC, size_t ldc,
                         unsigned nq, clblasQueue* queues, unsigned nev, const clblasEvent* wait, clblasEvent* events)
{
    return syrk_entry<double>(order, uplo, transA, N, K, alpha, A, offA, lda, beta, C, offC, ldc, nq, queues, nev, wait, events);
}

clblasStatus clblasSsyr2k(clblasOrder order, clblasUplo uplo, clblasTranspose transAB, size_t N, size_t K, float alpha,
                          const clblasMem A, size_t offA, size_t lda, const clblasMem B, size_t offB, size_t ldb, float beta,
                          clblasMem C, size_t offC, size_t ldc,
                          unsigned nq, clblasQueue* queues, unsigned nev, const clblasEvent* wait, clblasEvent* events)
{
    return syr2k_entry<float>(order, uplo, transAB, N, K, alpha, A, offA, lda, B, offB, ldb, beta, C, offC, ldc, nq, queues, nev, wait, events);
}

clblasStatus clblasDsyr2k(clblasOrder order, clblasUplo uplo, clblasTranspose transAB, size_t N, size_t K, double alpha,
                          const clblasMem A, size_t offA, size_t lda, const clblasMem B, size_t offB, size_t ldb, double beta,
                          clblasMem C, size_t offC, size_t ldc,
                          unsigned nq, clblasQueue* queues, unsigned nev, const clblasEvent* wait, clblasEvent* events)
{
    return syr2k_entry<double>(order, uplo, transAB, N, K, alpha, A, offA, lda, B, offB, ldb, beta, C, offC, ldc, nq, queues, nev, wait, events);
}

clblasStatus clblasSsymm(clblasOrder order, clblasSide side, clblasUplo uplo, size_t M, size_t N, float alpha,
                         const clblasMem A, size_t offa, size_t lda, const clblasMem B, size_t offb, size_t ldb, float beta,
                         clblasMem C, size_t offc, size_t ldc,
                         unsigned nq, clblasQueue* queues, unsigned nev, const clblasEvent* wait, clblasEvent* events)
{
    return symm_entry<float>(order, side, uplo, M, N, alpha, A, offa, lda, B, offb, ldb, beta, C, offc, ldc, nq, queues, nev, wait, events);
}

clblasStatus clblasDsymm(clblasOrder order, clblasSide side, clblasUplo uplo, size_t M, size_t N, double alpha,
                         const clblasMem A, size_t offa, size_t lda, const clblasMem B, size_t offb, size_t ldb, double beta,
                         clblasMem C, size_t offc, size_t ldc,
                         unsigned nq, clblasQueue* queues, unsigned nev, const clblasEvent* wait, clblasEvent* events)
{
    return symm_entry<double>(order, side, uplo, M, N, alpha, A, offa, lda, B, offb, ldb, beta, C, offc, ldc, nq, queues, nev, wait, events);
}

clblasStatus clblasCgemm(clblasOrder order, clblasTranspose transA, clblasTranspose transB, size_t M, size_t N, size_t K,
                         FloatComplex alpha, const clblasMem A, size_t offA, size_t lda, const clblasMem B, size_t offB, size_t ldb,
                         FloatComplex beta, clblasMem C, size_t offC, size_t ldc,
                         unsigned nq, clblasQueue* queues, unsigned nev, const clblasEvent* wait, clblasEvent* events)
{
    return cgemm_entry<float>(order, transA, transB, M, N, K, alpha.s[0], alpha.s[1], A, offA, lda, B, offB, ldb,
                              beta.s[0], beta.s[1], C, offC, ldc, nq, queues, nev, wait, events);
}

clblasStatus clblasZgemm(clblasOrder order, clblasTranspose transA, clblasTranspose transB, size_t M, size_t N, size_t K,
                         DoubleComplex alpha, const clblasMem A, size_t offA, size_t lda, const clblasMem B, size_t offB, size_t ldb,
                         DoubleComplex beta, clblasMem C, size_t offC, size_t ldc,
                         unsigned nq, clblasQueue* queues, unsigned nev, const clblasEvent* wait, clblasEvent* events)
{
    return cgemm_entry<double>(order, transA, transB, M, N, K, alpha.s[0], alpha.s[1], A, offA, lda, B, offB, ldb,
                               beta.s[0], beta.s[1], C, offC, ldc, nq, queues, nev, wait, events);
}

clblasStatus clblasCtrsm(clblasOrder order, clblasSide side, clblasUplo uplo, clblasTranspose transA, clblasDiag diag,
                         size_t M, size_t N, FloatComplex alpha, const clblasMem A, size_t offA, size_t lda,
                         clblasMem B, size_t offB, size_t ldb,
                         unsigned nq, clblasQueue* queues, unsigned nev, const clblasEvent* wait, clblasEvent* events)
{
    return ctrsm_entry<float>(order, side, uplo, transA, diag, M, N, alpha.s[0], alpha.s[1], A, offA, lda, B, offB, ldb,
                              nq, queues, nev, wait, events);
}

clblasStatus clblasZtrsm(clblasOrder order, clblasSide side, clblasUplo uplo, clblasTranspose transA, clblasDiag diag,
                         size_t M, size_t N, DoubleComplex alpha, const clblasMem A, size_t offA, size_t lda,
                         clblasMem B, size_t offB, size_t ldb,
                         unsigned nq, clblasQueue* queues, unsigned nev, const clblasEvent* wait, clblasEvent* events)
{
    return ctrsm_entry<double>(order, side, uplo, transA, diag, M, N, alpha.s[0], alpha.s[1], A, offA, lda, B, offB, ldb,
                               nq, queues, nev, wait, events);
}

clblasStatus clblasB200SgemmHost(clblasOrder order, clblasTranspose transA, clblasTranspose transB, size_t M, size_t N, size_t K,
                                 float alpha, const void* A, size_t offA, size_t lda, const void* B, size_t offB, size_t ldb,
                                 float beta, void* C, size_t offC, size_t ldc, unsigned nq, clblasQueue* queues,
                                 unsigned nev, const clblasEvent* wait, clblasEvent* events)
{
    return gemm_host_entry<float>(order, transA, transB, M, N, K, alpha, A, offA, lda, B, offB, ldb, beta, C, offC, ldc,
                                  nq, queues, nev, wait, events);
}

clblasStatus clblasB200DgemmHost(clblasOrder order, clblasTranspose transA, clblasTranspose transB, size_t M, size_t N, size_t K,
                                 double alpha, const void* A, size_t offA, size_t lda, const void* B, size_t offB, size_t ldb,
                                 double beta, void* C, size_t offC, size_t ldc, unsigned nq, clblasQueue* queues,
                                 unsigned nev, const clblasEvent* wait, clblasEvent* events)
{
    return gemm_host_entry<double>(order, transA, transB, M, N, K, alpha, A, offA, lda, B, offB, ldb, beta, C, offC, ldc,
                                   nq, queues, nev, wait, events);
}

clblasStatus clblasB200StrsmHost(clblasOrder order, clblasSide side, clblasUplo uplo, clblasTranspose transA, clblasDiag diag,
                                 size_t M, size_t N, float alpha, const void* A, size_t offA, size_t lda, void* B, size_t offB,
                                 size_t ldb, unsigned nq, clblasQueue* queues, unsigned nev, const clblasEvent* wait,
                                 clblasEvent* events)
{
    return trsm_host_entry<float>(order, side, uplo, transA, diag, M, N, alpha, A, offA, lda, B, offB, ldb, nq, queues, nev, wait, events);
}

clblasStatus clblasB200DtrsmHost(clblasOrder order, clblasSide side, clblasUplo uplo, clblasTranspose transA, clblasDiag diag,
                                 size_t M, size_t N, double alpha, const void* A, size_t offA, size_t lda, void* B, size_t offB,
                                 size_t ldb, unsigned nq, clblasQueue* queues, unsigned nev, const clblasEvent* wait,
                                 clblasEvent* events)
{
    return trsm_host_entry<double>(order, side, uplo, transA, diag, M, N, alpha, A, offA, lda, B, offB, ldb, nq, queues, nev, wait, events);
}

clblasStatus clblasCsyrk(clblasOrder order, clblasUplo uplo, clblasTranspose trans, size_t N, size_t K, FloatComplex alpha,
        const clblasMem A, size_t offA, size_t lda, FloatComplex beta, clblasMem C, size_t offC, size_t ldc,
        unsigned nq, clblasQueue* queues, unsigned nev, const clblasEvent* wait, clblasEvent* events)
{
    return csyrk_entry<float>(false, false, order, uplo, trans, N, K, alpha.s[0], alpha.s[1], A, offA, lda, nullptr, 0, 0, beta.s[0], beta.s[1],
                            C, offC, ldc, nq, queues, nev, wait, events);
}

clblasStatus clblasZsyrk(clblasOrder order, clblasUplo uplo, clblasTranspose trans, size_t N, size_t K, DoubleComplex alpha,
        const clblasMem A, size_t offA, size_t lda, DoubleComplex beta, clblasMem C, size_t offC, size_t ldc,
        unsigned nq, clblasQueue* queues, unsigned nev, const clblasEvent* wait, clblasEvent* events)
{
    return csyrk_entry<double>(false, false, order, uplo, trans, N, K, alpha.s[0], alpha.s[1], A, offA, lda, nullptr, 0, 0, beta.s[0], beta.s[1],
                            C, offC, ldc, nq, queues, nev, wait, events);
}

clblasStatus clblasCherk(clblasOrder order, clblasUplo uplo, clblasTranspose trans, size_t N, size_t K, float alpha,
        const clblasMem A, size_t offA, size_t lda, float beta, clblasMem C, size_t offC, size_t ldc,
        unsigned nq, clblasQueue* queues, unsigned nev, const clblasEvent* wait, clblasEvent* events)
{
    return csyrk_entry<float>(true, false, order, uplo, trans, N, K, alpha, (float)0, A, offA, lda, nullptr, 0, 0, beta, (float)0,
                            C, offC, ldc, nq, queues, nev, wait, events);
}

clblasStatus clblasZherk(clblasOrder order, clblasUplo uplo, clblasTranspose trans, size_t N, size_t K, double alpha,
        const clblasMem A, size_t offA, size_t lda, double beta, clblasMem C, size_t offC, size_t ldc,
        unsigned nq, clblasQueue* queues, unsigned nev, const clblasEvent* wait, clblasEvent* events)
{
    return csyrk_entry<double>(true, false, order, uplo, trans, N, K, alpha, (double)0, A, offA, lda, nullptr, 0, 0, beta, (double)0,
                            C, offC, ldc, nq, queues, nev, wait, events);
}

clblasStatus clblasCsyr2k(clblasOrder order, clblasUplo uplo, clblasTranspose trans, size_t N, size_t K, FloatComplex alpha,
        const clblasMem A, size_t offA, size_t lda, const clblasMem B, size_t offB, size_t ldb, FloatComplex beta, clblasMem C, size_t offC, size_t ldc,
        unsigned nq, clblasQueue* queues, unsigned nev, const clblasEvent* wait, clblasEvent* events)
{
    return csyrk_entry<float>(false, true, order, uplo, trans, N, K, alpha.s[0], alpha.s[1], A, offA, lda, B, offB, ldb, beta.s[0], beta.s[1],
                            C, offC, ldc, nq, queues, nev, wait, events);
}

clblasStatus clblasZsyr2k(clblasOrder order, clblasUplo uplo, clblasTranspose trans, size_t N, size_t K, DoubleComplex alpha,
        const clblasMem A, size_t offA, size_t lda, const clblasMem B, size_t offB, size_t ldb, DoubleComplex beta, clblasMem C, size_t offC, size_t ldc,
        unsigned nq, clblasQueue* queues, unsigned nev, const clblasEvent* wait, clblasEvent* events)
{
    return csyrk_entry<double>(false, true, order, uplo, trans, N, K, alpha.s[0], alpha.s[1], A, offA, lda, B, offB, ldb, beta.s[0], beta.s[1],
                            C, offC, ldc, nq, queues, nev, wait, events);
}

clblasStatus clblasCher2k(clblasOrder order, clblasUplo uplo, clblasTranspose trans, size_t N, size_t K, FloatComplex alpha,
        const clblasMem A, size_t offA, size_t lda, const clblasMem B, size_t offB, size_t ldb, float beta, clblasMem C, size_t offC, size_t ldc,
        unsigned nq, clblasQueue* queues, unsigned nev, const clblasEvent* wait, clblasEvent* events)
{
    return csyrk_entry<float>(true, true, order, uplo, trans, N, K, alpha.s[0], alpha.s[1], A, offA, lda, B, offB, ldb, beta, (float)0,
                            C, offC, ldc, nq, queues, nev, wait, events);
}

clblasStatus clblasZher2k(clblasOrder order, clblasUplo uplo, clblasTranspose trans, size_t N, size_t K, DoubleComplex alpha,
        const clblasMem A, size_t offA, size_t lda, const clblasMem B, size_t offB, size_t ldb, double beta, clblasMem C, size_t offC, size_t ldc,
        unsigned nq, clblasQueue* queues, unsigned nev, const clblasEvent* wait, clblasEvent* events)
{
    return csyrk_entry<double>(true, true, order, uplo, trans, N, K, alpha.s[0], alpha.s[1], A, offA, lda, B, offB, ldb, beta, (double)0,
                            C, offC, ldc, nq, queues, nev, wait, events);
}

clblasStatus clblasCsymm(clblasOrder order, clblasSide side, clblasUplo uplo, size_t M, size_t N, FloatComplex alpha,
        const clblasMem A, size_t offa, size_t lda, const clblasMem B, size_t offb, size_t ldb, FloatComplex beta,
        clblasMem C, size_t offc, size_t ldc,
        unsigned nq, clblasQueue* queues, unsigned nev, const clblasEvent* wait, clblasEvent* events)
{
    return csymm_entry<float>(false, order, side, uplo, M, N, alpha.s[0], alpha.s[1], A, offa, lda, B, offb, ldb,
                            beta.s[0], beta.s[1], C, offc, ldc, nq, queues, nev, wait, events);
}

clblasStatus clblasZsymm(clblasOrder order, clblasSide side, clblasUplo uplo, size_t M, size_t N, DoubleComplex alpha,
        const clblasMem A, size_t offa, size_t lda, const clblasMem B, size_t offb, size_t ldb, DoubleComplex beta,
        clblasMem C, size_t offc, size_t ldc,
        unsigned nq, clblasQueue* queues, unsigned nev, const clblasEvent* wait, clblasEvent* events)
{
    return csymm_entry<double>(false, order, side, uplo, M, N, alpha.s[0], alpha.s[1], A, offa, lda, B, offb, ldb,
                            beta.s[0], beta.s[1], C, offc, ldc, nq, queues, nev, wait, events);
}

clblasStatus clblasChemm(clblasOrder order, clblasSide side, clblasUplo uplo, size_t M, size_t N, FloatComplex alpha,
        const clblasMem A, size_t offa, size_t lda, const clblasMem B, size_t offb, size_t ldb, FloatComplex beta,
        clblasMem C, size_t offc, size_t ldc,
        unsigned nq, clblasQueue* queues, unsigned nev, const clblasEvent* wait, clblasEvent* events)
{
    return csymm_entry<float>(true, order, side, uplo, M, N, alpha.s[0], alpha.s[1], A, offa, lda, B, offb, ldb,
                            beta.s[0], beta.s[1], C, offc, ldc, nq, queues, nev, wait, events);
}

clblasStatus clblasZhemm(clblasOrder order, clblasSide side, clblasUplo uplo, size_t M, size_t N, DoubleComplex alpha,
        const clblasMem A, size_t offa, size_t lda, const clblasMem B, size_t offb, size_t ldb, DoubleComplex beta,
        clblasMem C, size_t offc, size_t ldc,
        unsigned nq, clblasQueue* queues, unsigned nev, const clblasEvent* wait, clblasEvent* events)
{
    return csymm_entry<double>(true, order, side, uplo, M, N, alpha.s[0], alpha.s[1], A, offa, lda, B, offb, ldb,
                            beta.s[0], beta.s[1], C, offc, ldc, nq, queues, nev, wait, events);
}

clblasStatus clblasCtrmm(clblasOrder order, clblasSide side, clblasUplo uplo, clblasTranspose transA, clblasDiag diag,
                         size_t M, size_t N, FloatComplex alpha, const clblasMem A, size_t offA, size_t lda,
                         clblasMem B, size_t offB, size_t ldb,
                         unsigned nq, clblasQueue* queues, unsigned nev, const clblasEvent* wait, clblasEvent* events)
{
    return ctrmm_entry<float>(order, side, uplo, transA, diag, M, N, alpha.s[0], alpha.s[1], A, offA, lda, B, offB, ldb,
                              nq, queues, nev, wait, events);
}

clblasStatus clblasZtrmm(clblasOrder order, clblasSide side, clblasUplo uplo, clblasTranspose transA, clblasDiag diag,
                         size_t M, size_t N, DoubleComplex alpha, const clblasMem A, size_t offA, size_t lda,
                         clblasMem B, size_t offB, size_t ldb,
                         unsigned nq, clblasQueue* queues, unsigned nev, const clblasEvent* wait, clblasEvent* events)
{
    return ctrmm_entry<double>(order, side, uplo, transA, diag, M, N, alpha.s[0], alpha.s[1], A, offA, lda, B, offB, ldb,
                               nq, queues, nev, wait, events);
}

clblasStatus clblasB200DtrsmNoAlloc(clblasOrder order, clblasSide side, clblasUplo uplo, clblasTranspose transA,
                                    clblasDiag diag, size_t M, size_t N, double alpha, const clblasMem A, size_t offA,
                                    size_t lda, clblasMem B, size_t offB, size_t ldb, unsigned nq, clblasQueue* queues,
                                    unsigned nev, const clblasEvent* wait, clblasEvent* events)
{
    // Same checks, in the same order, as clblasDtrsm; then the size limit of the fixed scratch array.
    clblasStatus st;
    if ((st = check_queues(nq, queues)) != clblasSuccess) return st;
    if ((st = check_events(nev, wait)) != clblasSuccess) return st;
    if (!g_initialized.load()) return clblasNotInitialized;
    if (A == nullptr) return clblasInvalidMatA;
    if (B == nullptr) return clblasInvalidMatB;
    if (order != clblasRowMajor && order != clblasColumnMajor) return clblasInvalidValue;
    if ((unsigned)side > 1u || (unsigned)uplo > 1u || (unsigned)transA > 2u || (unsigned)diag > 1u) return clblasInvalidValue;
    const size_t msize = (side == clblasLeft) ? M : N;
    if ((st = check_matrix_sizes(sizeof(double), order, transA, msize, msize, A, offA, lda, SET_A)) != clblasSuccess) return st;
    if ((st = check_matrix_sizes(sizeof(double), order, clblasNoTrans, M, N, B, offB, ldb, SET_B)) != clblasSuccess) return st;
    const size_t other = (side == clblasLeft) ? N : M;
    if (msize > CLBLAS_B200_NOALLOC_MAX_ORDER || other > CLBLAS_B200_NOALLOC_MAX_OTHER) return clblasOutOfResources;

    cudaStream_t s = reinterpret_cast<cudaStream_t>(queues[0]);
    if ((st = wait_all(s, nev, wait)) != clblasSuccess) return st;
    bool right = (side == clblasRight), lower = (uplo == clblasLower);
    if (order == clblasRowMajor) {
        size_t t = M; M = N; N = t;
        right = !right;
        lower = !lower;
    }
    cudaError_t e = dtrsm_colmajor_noalloc(right, lower, transA != clblasNoTrans, diag == clblasUnit, M, N, alpha,
                                           static_cast<const double*>(A) + offA, lda, static_cast<double*>(B) + offB, ldb, s);
    if (e != cudaSuccess) { cudaGetLastError(); return from_cuda(e); }
    return record_out(nq, queues, events);
}

clblasStatus clblasB200PlanShards(size_t total, unsigned parts, size_t align, size_t* bounds)
{
    if (parts == 0 || bounds == nullptr) return clblasInvalidValue;
    if (align == 0) align = 1;
    // Equal shares rounded up to the alignment; trailing devices may get less (or nothing).
    const size_t units = (total + align - 1) / align;
    const size_t per = (units + parts - 1) / parts;
    bounds[0] = 0;
    for (unsigned i = 1; i <= parts; i++) {
        size_t b = (size_t)i * per * align;
        bounds[i] = b < total ? b : total;
    }
    bounds[parts] = total;
    return clblasSuccess;
}

unsigned long long clblasB200LaunchCount(void) { return g_launches.load(); }

unsigned clblasB200DeviceFault(void)
{
    if (cudaDeviceSynchronize() != cudaSuccess) { cudaGetLastError(); return 0x80000000u; }
    return dgemm_tma_fault_flag() | sgemm_tma_fault_flag() | sgemm_3xtf32_fault_flag() | dtrsm_fused_fault_flag();
}
const char* clblasB200LastGemmKernel(void) { return t_last_kernel; }
const char* clblasB200LastGemmVariant(void) { return t_last_variant; }
unsigned long long clblasB200WorkspaceAllocCount(void) { return ws_alloc_count(); }
void clblasB200NoAllocLimits(size_t* max_order, size_t* max_other)
{
    if (max_order) *max_order = CLBLAS_B200_NOALLOC_MAX_ORDER;
    if (max_other) *max_other = CLBLAS_B200_NOALLOC_MAX_OTHER;
}

clblasStatus clblasB200SgemmSharded(clblasOrder order, clblasTranspose transA, clblasTranspose transB, size_t M, size_t N, size_t K,
                                    float alpha, clblasMem A, size_t offA, size_t lda, clblasMem B, size_t offB, size_t ldb,
                                    float beta, clblasMem C, size_t offC, size_t ldc, clblasB200Comm comm, int root,
                                    unsigned nq, clblasQueue* queues, unsigned nev, const clblasEvent* wait, clblasEvent* events)
{
    return gemm_sharded_entry<float>(order, transA, transB, M, N, K, alpha, A, offA, lda, B, offB, ldb, beta, C, offC, ldc,
                                     comm, root, nq, queues, nev, wait, events);
}

clblasStatus clblasB200DgemmSharded(clblasOrder order, clblasTranspose transA, clblasTranspose transB, size_t M, size_t N, size_t K,
                                    double alpha, clblasMem A, size_t offA, size_t lda, clblasMem B, size_t offB, size_t ldb,
                                    double beta, clblasMem C, size_t offC, size_t ldc, clblasB200Comm comm, int root,
                                    unsigned nq, clblasQueue* queues, unsigned nev, const clblasEvent* wait, clblasEvent* events)
{
    return gemm_sharded_entry<double>(order, transA, transB, M, N, K, alpha, A, offA, lda, B, offB, ldb, beta, C, offC, ldc,
                                      comm, root, nq, queues, nev, wait, events);
}

clblasStatus clblasB200StrsmSharded(clblasOrder order, clblasSide side, clblasUplo uplo, clblasTranspose transA, clblasDiag diag,
                                    size_t M, size_t N, float alpha, clblasMem A, size_t offA, size_t lda, clblasMem B, size_t offB,
                                    size_t ldb, clblasB200Comm comm, int root,
                                    unsigned nq, clblasQueue* queues, unsigned nev, const clblasEvent* wait, clblasEvent* events)
{
    return trsm_sharded_entry<float>(order, side, uplo, transA, diag, M, N, alpha, A, offA, lda, B, offB, ldb, comm, root,
                                     nq, queues, nev, wait, events);
}

clblasStatus clblasB200DtrsmSharded(clblasOrder order, clblasSide side, clblasUplo uplo, clblasTranspose transA, clblasDiag diag,
                                    size_t M, size_t N, double alpha, clblasMem A, size_t offA, size_t lda, clblasMem B, size_t offB,
                                    size_t ldb, clblasB200Comm comm, int root,
                                    unsigned nq, clblasQueue* queues, unsigned nev, const clblasEvent* wait, clblasEvent* events)
{
    return trsm_sharded_entry<double>(order, side, uplo, transA, diag, M, N, alpha, A, offA, lda, B, offB, ldb, comm, root,
                                      nq, queues, nev, wait, events);
}
int clblasB200SetGemmPath(int path) { return g_forced_path.exchange(path); }

}  // extern "C"
