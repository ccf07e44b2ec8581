/*
 * clblas_b200.h -- C ABI of the B200 (sm_100a) level-3 hot path behind the clBLAS call shape.
 *
 * Every entry point below keeps the argument list of the clBLAS function it replaces
 * (reference header src/clBLAS.h).  The OpenCL handle types are mapped one-to-one:
 *
 *     cl_mem            ->  clblasMem    (void*, a CUDA device pointer)
 *     cl_command_queue  ->  clblasQueue  (cudaStream_t)
 *     cl_event          ->  clblasEvent  (cudaEvent_t)
 *     cl_uint/cl_float/cl_double -> unsigned/float/double
 *
 * Offsets are counted in elements, exactly as in the reference (src/clBLAS.h:7345-7346).
 * Errors are reported only through the returned clblasStatus; no exception crosses this ABI.
 * The library has no CPU code path: every call either launches CUDA kernels on the stream it
 * was given or returns an error status.
 */
#ifndef CLBLAS_B200_H_
#define CLBLAS_B200_H_

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void*               clblasMem;
typedef struct CUstream_st* clblasQueue;
typedef struct CUevent_st*  clblasEvent;

/* Enumerations: same names and the same numeric values as src/clBLAS.h:78-113. */
/* Complex scalars and matrix elements: (re, im) pairs with the layout, size and alignment of the reference's
 * FloatComplex / DoubleComplex (cl_float2 / cl_double2, src/clBLAS-complex.h:27-58), passed by value. */
#if defined(__GNUC__) || defined(__clang__) || defined(__CUDACC__)
#define CLBLAS_B200_ALIGNED(n) __attribute__((aligned(n)))
#else
#define CLBLAS_B200_ALIGNED(n)
#endif
typedef struct CLBLAS_B200_ALIGNED(8)  { float s[2]; }  FloatComplex;
typedef struct CLBLAS_B200_ALIGNED(16) { double s[2]; } DoubleComplex;
static inline FloatComplex floatComplex(float real, float imag) { FloatComplex z; z.s[0] = real; z.s[1] = imag; return z; }
static inline DoubleComplex doubleComplex(double real, double imag) { DoubleComplex z; z.s[0] = real; z.s[1] = imag; return z; }
#define CREAL(v) ((v).s[0])
#define CIMAG(v) ((v).s[1])

typedef enum clblasOrder_     { clblasRowMajor = 0, clblasColumnMajor = 1 } clblasOrder;
typedef enum clblasTranspose_ { clblasNoTrans = 0, clblasTrans = 1, clblasConjTrans = 2 } clblasTranspose;
typedef enum clblasUplo_      { clblasUpper = 0, clblasLower = 1 } clblasUplo;
typedef enum clblasDiag_      { clblasUnit = 0, clblasNonUnit = 1 } clblasDiag;
typedef enum clblasSide_      { clblasLeft = 0, clblasRight = 1 } clblasSide;

/* Status codes: same names and values as src/clBLAS.h:123-155.  The first block aliases
 * OpenCL error numbers there; the numbers are the OpenCL specification's constants. */
typedef enum clblasStatus_ {
    clblasSuccess               = 0,
    clblasInvalidValue          = -30,
    clblasInvalidCommandQueue   = -36,
    clblasInvalidContext        = -34,
    clblasInvalidMemObject      = -38,
    clblasInvalidDevice         = -33,
    clblasInvalidEventWaitList  = -57,
    clblasOutOfResources        = -5,
    clblasOutOfHostMemory       = -6,
    clblasInvalidOperation      = -59,
    clblasCompilerNotAvailable  = -3,
    clblasBuildProgramFailure   = -11,
    clblasNotImplemented        = -1024,
    clblasNotInitialized        = -1023,
    clblasInvalidMatA           = -1022,
    clblasInvalidMatB           = -1021,
    clblasInvalidMatC           = -1020,
    clblasInvalidVecX           = -1019,
    clblasInvalidVecY           = -1018,
    clblasInvalidDim            = -1017,
    clblasInvalidLeadDimA       = -1016,
    clblasInvalidLeadDimB       = -1015,
    clblasInvalidLeadDimC       = -1014,
    clblasInvalidIncX           = -1013,
    clblasInvalidIncY           = -1012,
    clblasInsufficientMemMatA   = -1011,
    clblasInsufficientMemMatB   = -1010,
    clblasInsufficientMemMatC   = -1009,
    clblasInsufficientMemVecX   = -1008,
    clblasInsufficientMemVecY   = -1007
} clblasStatus;

/* ---- life cycle: replaces src/clBLAS.h:176-213 (src/library/blas/init.c:34-263) ---------- */

/* Version of the clBLAS API this library is a drop-in for (2.12.0, src/CMakeLists.txt:107-118). */
clblasStatus clblasGetVersion(unsigned* major, unsigned* minor, unsigned* patch);
/* Idempotent; creates per-device state lazily.  Not thread safe (src/clBLAS.h:59-61). */
clblasStatus clblasSetup(void);
/* Releases cached per-device state (TRSM workspaces). */
void clblasTeardown(void);

/* ---- GEMM: replaces clblasSgemm (src/clBLAS.h:7382-7405) and clblasDgemm (:7463-7486),
 *      implemented by src/library/blas/xgemm.cc:341-783 in the reference.
 *      C <- alpha*op(A)*op(B) + beta*C.  Row-major is served by the reference's operand swap
 *      (xgemm.cc:40-61); ConjTrans means Trans for real types (xgemm.cc:330-335).
 *      Argument checks, in the reference's order (xgemm.cc:685-706, generic/common.c:585-686):
 *      NULL A/B/C -> InvalidMat{A,B,C}; if K != 0: A then B sizes; always C sizes;
 *      M == 0 or N == 0 -> InvalidDim; short ld -> InvalidLeadDim{A,B,C}; matrix extent beyond
 *      the CUDA allocation holding the pointer -> InsufficientMemMat{A,B,C}.
 *      numCommandQueues >= 1.  With one queue the whole product runs on it.  With several, N is cut into
 *      one stripe per queue, boundaries multiples of 128, and stripe q runs on commandQueues[q] -- what the
 *      reference's multi-queue GEMM does (xgemm.cc:603-658; stripes of
 *      src/library/blas/generic/solution_seq_make.c:764-866).  The matrices live on the device of
 *      commandQueues[0]; a queue on another device of the same process is given copies of A and of its
 *      stripes of B and C, and its stripe of C is copied back before its event is recorded (OpenCL queues
 *      of one context share their buffers, GPUs do not).  Every other level-3 routine of this library does
 *      its work on commandQueues[0], as the reference's TRSM does (src/library/blas/xtrsm.cc:1626-1629).
 *      The call is asynchronous: work is ordered after every event of eventWaitList and, when
 *      events != NULL, every non-NULL events[q] (q < numCommandQueues) must be a created cudaEvent_t; it
 *      is recorded on commandQueues[q] when the work that queue has to wait for is complete. */
clblasStatus clblasSgemm(
    clblasOrder order, clblasTranspose transA, clblasTranspose transB,
    size_t M, size_t N, size_t K,
    float alpha,
    const clblasMem A, size_t offA, size_t lda,
    const clblasMem B, size_t offB, size_t ldb,
    float beta,
    clblasMem C, size_t offC, size_t ldc,
    unsigned numCommandQueues, clblasQueue* commandQueues,
    unsigned numEventsInWaitList, const clblasEvent* eventWaitList, clblasEvent* events);

clblasStatus clblasDgemm(
    clblasOrder order, clblasTranspose transA, clblasTranspose transB,
    size_t M, size_t N, size_t K,
    double alpha,
    const clblasMem A, size_t offA, size_t lda,
    const clblasMem B, size_t offB, size_t ldb,
    double beta,
    clblasMem C, size_t offC, size_t ldc,
    unsigned numCommandQueues, clblasQueue* commandQueues,
    unsigned numEventsInWaitList, const clblasEvent* eventWaitList, clblasEvent* events);

/* ---- complex GEMM: replaces clblasCgemm (src/clBLAS.h:7538-7560) and clblasZgemm (:7614-7636), which the
 *      reference serves through the same clblasGemm<T> front end (src/library/blas/xgemm.cc:788-905): same
 *      checks in the same order as the real routines.  Matrices hold interleaved (re, im) pairs; offsets and
 *      leading dimensions count complex elements; clblasConjTrans conjugates.  Takes a workspace of about
 *      twice the size of A (plus the size of B when B is transposed) from the library's pool. */
clblasStatus clblasCgemm(
    clblasOrder order, clblasTranspose transA, clblasTranspose transB,
    size_t M, size_t N, size_t K,
    FloatComplex alpha,
    const clblasMem A, size_t offA, size_t lda,
    const clblasMem B, size_t offB, size_t ldb,
    FloatComplex beta,
    clblasMem C, size_t offC, size_t ldc,
    unsigned numCommandQueues, clblasQueue* commandQueues,
    unsigned numEventsInWaitList, const clblasEvent* eventWaitList, clblasEvent* events);

clblasStatus clblasZgemm(
    clblasOrder order, clblasTranspose transA, clblasTranspose transB,
    size_t M, size_t N, size_t K,
    DoubleComplex alpha,
    const clblasMem A, size_t offA, size_t lda,
    const clblasMem B, size_t offB, size_t ldb,
    DoubleComplex beta,
    clblasMem C, size_t offC, size_t ldc,
    unsigned numCommandQueues, clblasQueue* commandQueues,
    unsigned numEventsInWaitList, const clblasEvent* eventWaitList, clblasEvent* events);

/* ---- TRSM: replaces clblasStrsm (src/clBLAS.h:7988-8008, src/library/blas/xtrsm.cc:1601-1661)
 *      and clblasDtrsm (src/clBLAS.h:8063-8083, xtrsm.cc:1664-1785, blocked algorithm :1136-1507).
 *      Solves op(A)*X = alpha*B (Left) or X*op(A) = alpha*B (Right); X overwrites B.
 *      Checks follow the reference's STRSM order (xtrsm.cc:1623-1624,
 *      functor/functor_xtrsm.cc:57-75): queues, events, NotInitialized (clblasSetup not called),
 *      NULL A/B, A sizes (order x order), B sizes.  Row-major is served by the side/uplo flip of
 *      xtrsm.cc:54-64 for both precisions.  The out-of-triangle part of A is never read. */
clblasStatus clblasStrsm(
    clblasOrder order, clblasSide side, clblasUplo uplo, clblasTranspose transA, clblasDiag diag,
    size_t M, size_t N,
    float alpha,
    const clblasMem A, size_t offA, size_t lda,
    clblasMem B, size_t offB, size_t ldb,
    unsigned numCommandQueues, clblasQueue* commandQueues,
    unsigned numEventsInWaitList, const clblasEvent* eventWaitList, clblasEvent* events);

clblasStatus clblasDtrsm(
    clblasOrder order, clblasSide side, clblasUplo uplo, clblasTranspose transA, clblasDiag diag,
    size_t M, size_t N,
    double alpha,
    const clblasMem A, size_t offA, size_t lda,
    clblasMem B, size_t offB, size_t ldb,
    unsigned numCommandQueues, clblasQueue* commandQueues,
    unsigned numEventsInWaitList, const clblasEvent* eventWaitList, clblasEvent* events);

/* ---- complex TRSM: replaces clblasCtrsm (src/clBLAS.h:8132-8151) and clblasZtrsm (:8202-8221), which the
 *      reference serves through the same front end and checks as clblasStrsm (src/library/blas/xtrsm.cc:1787-1911,
 *      functor/functor_xtrsm.cc:57-75).  Interleaved (re, im) matrices; clblasConjTrans conjugates.  Workspace
 *      from the library's pool: about twice the size of A, plus a copy of B for side == clblasRight. */
clblasStatus clblasCtrsm(
    clblasOrder order, clblasSide side, clblasUplo uplo, clblasTranspose transA, clblasDiag diag,
    size_t M, size_t N,
    FloatComplex alpha,
    const clblasMem A, size_t offA, size_t lda,
    clblasMem B, size_t offB, size_t ldb,
    unsigned numCommandQueues, clblasQueue* commandQueues,
    unsigned numEventsInWaitList, const clblasEvent* eventWaitList, clblasEvent* events);

clblasStatus clblasZtrsm(
    clblasOrder order, clblasSide side, clblasUplo uplo, clblasTranspose transA, clblasDiag diag,
    size_t M, size_t N,
    DoubleComplex alpha,
    const clblasMem A, size_t offA, size_t lda,
    clblasMem B, size_t offB, size_t ldb,
    unsigned numCommandQueues, clblasQueue* commandQueues,
    unsigned numEventsInWaitList, const clblasEvent* eventWaitList, clblasEvent* events);

/* ---- TRMM: replaces clblasStrmm (src/clBLAS.h:7697-7717) and clblasDtrmm (:7772-7792), implemented by
 *      src/library/blas/xtrmm.c:30-180 in the reference.  B <- alpha*op(A)*B (Left) or alpha*B*op(A) (Right),
 *      A triangular; only the referenced triangle is read and a unit diagonal is not read.  Checks in the
 *      order of the reference's doTrmm (xtrmm.c:52-70): NotInitialized, NULL A/B, A sizes, B sizes.
 *      Needs clblasSetup(); takes its workspace from the library's stream-ordered pool. */
clblasStatus clblasStrmm(
    clblasOrder order, clblasSide side, clblasUplo uplo, clblasTranspose transA, clblasDiag diag,
    size_t M, size_t N,
    float alpha,
    const clblasMem A, size_t offA, size_t lda,
    clblasMem B, size_t offB, size_t ldb,
    unsigned numCommandQueues, clblasQueue* commandQueues,
    unsigned numEventsInWaitList, const clblasEvent* eventWaitList, clblasEvent* events);

clblasStatus clblasDtrmm(
    clblasOrder order, clblasSide side, clblasUplo uplo, clblasTranspose transA, clblasDiag diag,
    size_t M, size_t N,
    double alpha,
    const clblasMem A, size_t offA, size_t lda,
    clblasMem B, size_t offB, size_t ldb,
    unsigned numCommandQueues, clblasQueue* commandQueues,
    unsigned numEventsInWaitList, const clblasEvent* eventWaitList, clblasEvent* events);

/* ---- SYRK: replaces clblasSsyrk (src/clBLAS.h:8279-8296) and clblasDsyrk (:8351-8368), implemented by
 *      src/library/blas/xsyrk.c in the reference.  C <- alpha*op(A)*op(A)^T + beta*C on the `uplo` triangle of
 *      the N x N matrix C, op(A) N x K; the other triangle of C is neither read nor written.  Checks in the
 *      reference's order (xsyrk.c:48-70): NotInitialized, queues (InvalidValue), NULL A/C, A sizes, C sizes. */
clblasStatus clblasSsyrk(
    clblasOrder order, clblasUplo uplo, clblasTranspose transA,
    size_t N, size_t K,
    float alpha,
    const clblasMem A, size_t offA, size_t lda,
    float beta,
    clblasMem C, size_t offC, size_t ldc,
    unsigned numCommandQueues, clblasQueue* commandQueues,
    unsigned numEventsInWaitList, const clblasEvent* eventWaitList, clblasEvent* events);

clblasStatus clblasDsyrk(
    clblasOrder order, clblasUplo uplo, clblasTranspose transA,
    size_t N, size_t K,
    double alpha,
    const clblasMem A, size_t offA, size_t lda,
    double beta,
    clblasMem C, size_t offC, size_t ldc,
    unsigned numCommandQueues, clblasQueue* commandQueues,
    unsigned numEventsInWaitList, const clblasEvent* eventWaitList, clblasEvent* events);

/* ---- SYR2K: replaces clblasSsyr2k (src/clBLAS.h:8568-8589) and clblasDsyr2k (:8648-8669), implemented by
 *      src/library/blas/xsyr2k.c in the reference.  C <- alpha*op(A)*op(B)^T + alpha*op(B)*op(A)^T + beta*C on the
 *      `uplo` triangle of the N x N matrix C; op(A), op(B) are N x K.  Checks in the reference's order
 *      (xsyr2k.c:52-78): NotInitialized, queues (InvalidValue), NULL A/B/C, A sizes, B sizes, C sizes. */
clblasStatus clblasSsyr2k(
    clblasOrder order, clblasUplo uplo, clblasTranspose transAB,
    size_t N, size_t K,
    float alpha,
    const clblasMem A, size_t offA, size_t lda,
    const clblasMem B, size_t offB, size_t ldb,
    float beta,
    clblasMem C, size_t offC, size_t ldc,
    unsigned numCommandQueues, clblasQueue* commandQueues,
    unsigned numEventsInWaitList, const clblasEvent* eventWaitList, clblasEvent* events);

clblasStatus clblasDsyr2k(
    clblasOrder order, clblasUplo uplo, clblasTranspose transAB,
    size_t N, size_t K,
    double alpha,
    const clblasMem A, size_t offA, size_t lda,
    const clblasMem B, size_t offB, size_t ldb,
    double beta,
    clblasMem C, size_t offC, size_t ldc,
    unsigned numCommandQueues, clblasQueue* commandQueues,
    unsigned numEventsInWaitList, const clblasEvent* eventWaitList, clblasEvent* events);

/* ---- SYMM: replaces clblasSsymm (src/clBLAS.h:8898-8919) and clblasDsymm (:8979-9000), implemented by
 *      src/library/blas/xsymm.c in the reference.  C <- alpha*A*B + beta*C (Left, A M x M) or alpha*B*A + beta*C
 *      (Right, A N x N); A is symmetric and only its `uplo` triangle is read.  Checks in the reference's order
 *      (xsymm.c doSymm): NotInitialized, NULL A/B/C, A sizes, B sizes, C sizes, queues (InvalidValue), wait list.
 *      Takes an n x n workspace (n the order of A) from the library's stream-ordered pool. */
clblasStatus clblasSsymm(
    clblasOrder order, clblasSide side, clblasUplo uplo,
    size_t M, size_t N,
    float alpha,
    const clblasMem A, size_t offa, size_t lda,
    const clblasMem B, size_t offb, size_t ldb,
    float beta,
    clblasMem C, size_t offc, size_t ldc,
    unsigned numCommandQueues, clblasQueue* commandQueues,
    unsigned numEventsInWaitList, const clblasEvent* eventWaitList, clblasEvent* events);

clblasStatus clblasDsymm(
    clblasOrder order, clblasSide side, clblasUplo uplo,
    size_t M, size_t N,
    double alpha,
    const clblasMem A, size_t offa, size_t lda,
    const clblasMem B, size_t offb, size_t ldb,
    double beta,
    clblasMem C, size_t offc, size_t ldc,
    unsigned numCommandQueues, clblasQueue* commandQueues,
    unsigned numEventsInWaitList, const clblasEvent* eventWaitList, clblasEvent* events);

/* ---- DTRSM that allocates nothing (no counterpart in the reference, whose DTRSM creates and
 *      releases two OpenCL buffers inside every call, src/library/blas/xtrsm.cc:1183-1207).
 *      Same arguments, checks and result as clblasDtrsm, but the blocked solve's workspace is a
 *      fixed 12 MiB array that lives in device memory for as long as the library is loaded, so the
 *      call makes no cudaMalloc / cudaMallocAsync / cudaFree of any kind.  It is meant for callers
 *      that must not allocate while running: a server that gave all device memory to its own pool
 *      at start-up, or a loop with a fixed memory budget where an allocation that stalls or fails
 *      is not acceptable.
 *      Limits: order of A (M for Left, N for Right) <= CLBLAS_B200_NOALLOC_MAX_ORDER and the other
 *      dimension of B <= CLBLAS_B200_NOALLOC_MAX_OTHER; larger problems return
 *      clblasOutOfResources and touch nothing.
 *      The first call on each device does all the one-time work the entry point can ever need there: it
 *      looks up the array's device address, and it sets the shared-memory attribute of, and loads, every
 *      kernel a later call may dispatch to, whatever that call's transposition, width or alignment.  Make that
 *      first call before starting any stream capture.
 *      Every call on a device uses the same array: calls that may overlap on the GPU (streams with
 *      no ordering between them) race and give wrong results -- order them on one stream or with
 *      events.  What an earlier call left in the array never influences a later one. */
#define CLBLAS_B200_NOALLOC_MAX_ORDER 4096
#define CLBLAS_B200_NOALLOC_MAX_OTHER 8192
clblasStatus clblasB200DtrsmNoAlloc(
    clblasOrder order, clblasSide side, clblasUplo uplo, clblasTranspose transA, clblasDiag diag,
    size_t M, size_t N,
    double alpha,
    const clblasMem A, size_t offA, size_t lda,
    clblasMem B, size_t offB, size_t ldb,
    unsigned numCommandQueues, clblasQueue* commandQueues,
    unsigned numEventsInWaitList, const clblasEvent* eventWaitList, clblasEvent* events);

/* ---- partition planning: replaces the per-queue problem split of
 *      src/library/blas/generic/solution_seq_make.c:764-866 (stripeDivision over the N
 *      dimension, pieces aligned to DIVISION_ALIGNMENT = 128).
 *      Splits `total` columns over `parts` devices in contiguous blocks whose boundaries are
 *      multiples of `align` (the last block takes the remainder).  Writes parts+1 boundaries to
 *      `bounds` (bounds[0] = 0, bounds[parts] = total).  Pure host arithmetic; no CUDA call. */
clblasStatus clblasB200PlanShards(size_t total, unsigned parts, size_t align, size_t* bounds);

/* ---- one process (or thread) per GPU: the sharded forms.  They replace, for GPUs that do not share
 *      buffers, the reference's "one SolutionStep per command queue" execution
 *      (src/library/blas/generic/solution_seq_make.c:371-419, stripes :764-866) and the round-robin
 *      queue use of its GEMM (src/library/blas/xgemm.cc:603-658).
 *
 *      A communicator joins `nranks` GPUs of one box.  NCCL carries the traffic and is loaded at run
 *      time (dlopen of libnccl.so.2; a copy already mapped by the process is preferred; the environment
 *      variable CLBLAS_B200_NCCL_LIB names another); without it these calls return clblasNotImplemented.
 *      clblasB200CommGetUniqueId: one rank obtains 128 bytes and hands them to the others by any means.
 *      clblasB200CommInitRank: collective; call it with the rank's device current.  nranks == 1 needs no id.
 *      clblasB200CommInitAll: all ranks of one process at once (devices == NULL: devices 0..ndev-1), for a
 *      program that drives each GPU from its own thread.
 *      clblasB200CommDestroy: collective in effect (every rank destroys its end). */
#define CLBLAS_B200_UNIQUE_ID_BYTES 128
typedef void* clblasB200Comm;
clblasStatus clblasB200CommGetUniqueId(void* id128);
clblasStatus clblasB200CommInitRank(clblasB200Comm* comm, const void* id128, int nranks, int rank);
clblasStatus clblasB200CommInitAll(clblasB200Comm* comms, int ndev, const int* devices);
clblasStatus clblasB200CommDestroy(clblasB200Comm comm);
clblasStatus clblasB200CommInfo(clblasB200Comm comm, int* nranks, int* rank);

/*      clblasB200{S,D}gemmSharded: the argument list of clblasSgemm / clblasDgemm on ONE RANK'S SHARD, plus
 *      the communicator and the root rank.  Column-major: N is the number of columns of op(B) and C this rank
 *      owns (B and C point at the rank's own column block; boundaries as clblasB200PlanShards gives them;
 *      N == 0 is legal); A is the whole matrix on the root and a buffer of the same extent
 *      (same lda) on every other rank, which the call fills: A is broadcast in column panels of the matrix
 *      as stored, on a second stream, and the product of panel p starts when panel p has arrived, so the
 *      transfer of later panels overlaps the products (transA == NoTrans: K slabs accumulated with beta on
 *      the first and 1 afterwards, the reference's K split,
 *      src/library/blas/specialCases/GemmSpecialCases.cpp:127-191; otherwise blocks of rows of C).
 *      Row-major: the roles swap with the operands (src/library/blas/xgemm.cc:40-61): M counts the rank's
 *      rows of op(A) and C, and B is the broadcast matrix.
 *      M, K, alpha, the transpositions, the layout of the broadcast matrix and `root` must agree on all
 *      ranks; every rank of the communicator must make the call.  comm == NULL or a communicator of one
 *      rank: a plain GEMM.  Checks and status codes as clblasSgemm.  Work is issued on commandQueues[0]
 *      (and the communicator's own stream); the call is asynchronous like every other one. */
clblasStatus clblasB200SgemmSharded(
    clblasOrder order, clblasTranspose transA, clblasTranspose transB,
    size_t M, size_t N, size_t K,
    float alpha,
    clblasMem A, size_t offA, size_t lda,
    clblasMem B, size_t offB, size_t ldb,
    float beta,
    clblasMem C, size_t offC, size_t ldc,
    clblasB200Comm comm, int root,
    unsigned numCommandQueues, clblasQueue* commandQueues,
    unsigned numEventsInWaitList, const clblasEvent* eventWaitList, clblasEvent* events);

clblasStatus clblasB200DgemmSharded(
    clblasOrder order, clblasTranspose transA, clblasTranspose transB,
    size_t M, size_t N, size_t K,
    double alpha,
    clblasMem A, size_t offA, size_t lda,
    clblasMem B, size_t offB, size_t ldb,
    double beta,
    clblasMem C, size_t offC, size_t ldc,
    clblasB200Comm comm, int root,
    unsigned numCommandQueues, clblasQueue* commandQueues,
    unsigned numEventsInWaitList, const clblasEvent* eventWaitList, clblasEvent* events);

/*      clblasB200{S,D}trsmSharded: the argument list of clblasStrsm / clblasDtrsm on one rank's shard of the
 *      right-hand sides: the dimension of B that is not the order of A (N for Left, M for Right) counts what
 *      this rank owns (zero is legal) and B points at the rank's own block.  A is the whole triangular matrix
 *      on the root and a buffer of the same extent elsewhere; it is broadcast in column panels (a first one of 1/32 of the
 *      columns where the substitution starts, each next one four times as wide) in the order the substitution reaches them, and each step of the blocked solve waits
 *      only for the panels it reads, so the solve starts after the first panel and the rest of the transfer is
 *      hidden behind it.  No other exchange takes place: right-hand sides are independent
 *      (the reference's split, src/library/blas/generic/solution_seq_make.c:785-866). */
clblasStatus clblasB200StrsmSharded(
    clblasOrder order, clblasSide side, clblasUplo uplo, clblasTranspose transA, clblasDiag diag,
    size_t M, size_t N,
    float alpha,
    clblasMem A, size_t offA, size_t lda,
    clblasMem B, size_t offB, size_t ldb,
    clblasB200Comm comm, int root,
    unsigned numCommandQueues, clblasQueue* commandQueues,
    unsigned numEventsInWaitList, const clblasEvent* eventWaitList, clblasEvent* events);

clblasStatus clblasB200DtrsmSharded(
    clblasOrder order, clblasSide side, clblasUplo uplo, clblasTranspose transA, clblasDiag diag,
    size_t M, size_t N,
    double alpha,
    clblasMem A, size_t offA, size_t lda,
    clblasMem B, size_t offB, size_t ldb,
    clblasB200Comm comm, int root,
    unsigned numCommandQueues, clblasQueue* commandQueues,
    unsigned numEventsInWaitList, const clblasEvent* eventWaitList, clblasEvent* events);

/*      The panel plans the sharded calls use for a matrix of `columns` stored columns.  min_columns > 0 (products):
 *      a first panel of about 1/32 of the columns (at least min_columns), each next one four times as wide,
 *      boundaries multiples of 128, at most max_panels panels.  min_columns 0 / 1 (triangular solves whose substitution
 *      starts at the first / at the last column; max_panels >= 10): the same growth from a first panel of at least 128
 *      columns, the small panels at the end the substitution starts from.  Writes count+1 boundaries (bounds needs
 *      max_panels+1 entries).  Pure host arithmetic, exported for the tests. */
clblasStatus clblasB200PanelPlan(size_t columns, size_t min_columns, unsigned max_panels, size_t* bounds, unsigned* count);

/* ---- introspection used by the benchmark client and the tests (no reference counterpart
 *      beyond the AUTOGEMM_PRINT_DEBUG kernel-name print of xgemm.cc:437-445) ------------- */

/* Number of CUDA kernels this library has launched in the calling process so far. */
unsigned long long clblasB200LaunchCount(void);
/* Synchronises the current device and returns 0 when no kernel of this library ever gave up a
 * bounded wait on it (every in-kernel wait on an mbarrier has an iteration limit; a kernel whose
 * wait runs out sets a sticky flag and returns instead of hanging).  Non-zero = results of
 * earlier calls on this device are not to be trusted. */
unsigned clblasB200DeviceFault(void);
/* Issue-rate probe of the current device: kind 0 = FP32 FMA pipe, kind 1 = FP64 tensor-core
 * (mma.sync m8n8k4) pipe.  Runs register-only FMA/MMA loops for about `seconds` and returns the best
 * TFLOP/s seen (negative on error).  The benchmark uses it as the live roofline denominator. */
double clblasB200ProbePeak(int kind, double seconds);
/* Name of the kernel family the most recent GEMM of the calling thread dispatched to
 * ("dgemm_mma_tma", "sgemm_ffma_tma", "gemm_simt_ldg", ...).  Static storage; never NULL. */
const char* clblasB200LastGemmKernel(void);
/* The instantiation and mode behind that name, e.g. "dgemm_mma_tma<T,N,128>+streamk_tail",
 * "sgemm_ffma_tma<N,N,64,3,2>+splitk2", "sgemm_nt_16x8+tri": lets a test assert which variant it exercised.
 * Thread-local storage, overwritten by the thread's next GEMM; never NULL. */
const char* clblasB200LastGemmVariant(void);
/* Number of workspace allocations the level-3 routines of this library have made in the calling process so far
 * (operand repacking, split-K and stream-K partial tiles, TRSM's inverted blocks ...).  A call across which the
 * number does not change allocated nothing. */
unsigned long long clblasB200WorkspaceAllocCount(void);
/* The two size limits of clblasB200DtrsmNoAlloc as the built library has them (= the macros above). */
void clblasB200NoAllocLimits(size_t* max_order, size_t* max_other);
/* Forces a kernel family for GEMM calls of the whole process: 0 = automatic dispatch,
 * 1 = always the alignment-free LDG path, 2 / 3 = SGEMM TMA path with one / two CTAs per SM
 * (tuning aid; operands the TMA path cannot address still take the LDG path),
 * 4 = SGEMM through the optional 3xTF32 tensor-core kernel (tcgen05): each FP32 operand is split into
 * two TF32 numbers and three tensor-core products are accumulated in FP32; the result meets the
 * library's SGEMM tolerance (4*K*2^-24 relative to |alpha||A||B| + |beta||C|) but is not bit-identical to
 * the default FFMA kernel, hence opt-in.  The environment variable CLBLAS_B200_GEMM_PATH, read by
 * clblasSetup(), sets the same switch (the reference's counterpart: AMD_CLBLAS_GEMM_IMPLEMENTATION,
 * src/library/blas/impl.c:81-129).  Returns the previous value. */
int clblasB200SetGemmPath(int path);

/* ---- complex TRMM: replaces clblasCtrmm (src/clBLAS.h:7839) and clblasZtrmm (:7909); same checks as clblasStrmm.
 *      B <- alpha*op(A)*B (Left) or alpha*B*op(A) (Right), A triangular, interleaved (re, im) matrices;
 *      clblasConjTrans conjugates. */
clblasStatus clblasCtrmm(
    clblasOrder order, clblasSide side, clblasUplo uplo, clblasTranspose transA, clblasDiag diag,
    size_t M, size_t N,
    FloatComplex alpha,
    const clblasMem A, size_t offA, size_t lda,
    clblasMem B, size_t offB, size_t ldb,
    unsigned numCommandQueues, clblasQueue* commandQueues,
    unsigned numEventsInWaitList, const clblasEvent* eventWaitList, clblasEvent* events);

clblasStatus clblasZtrmm(
    clblasOrder order, clblasSide side, clblasUplo uplo, clblasTranspose transA, clblasDiag diag,
    size_t M, size_t N,
    DoubleComplex alpha,
    const clblasMem A, size_t offA, size_t lda,
    clblasMem B, size_t offB, size_t ldb,
    unsigned numCommandQueues, clblasQueue* commandQueues,
    unsigned numEventsInWaitList, const clblasEvent* eventWaitList, clblasEvent* events);

/* ---- complex symmetric / Hermitian level-3: replace clblasCsyrk / Zsyrk (src/clBLAS.h:8417, :8485), clblasCherk / Zherk
 *      (:9389, :9458; real alpha and beta), clblasCsyr2k / Zsyr2k (:8722, :8798), clblasCher2k / Zher2k (:9545, :9623;
 *      real beta), clblasCsymm / Zsymm (:9052, :9124) and clblasChemm / Zhemm (:9224, :9305); reference front ends
 *      src/library/blas/xsyrk.c, xherk.c, xsyr2k.c, xher2k.c, xsymm.c, xhemm.c.  Same checks in the same order; a
 *      symmetric update refuses clblasConjTrans and a Hermitian one clblasTrans (clblasInvalidValue).  Only the
 *      `uplo` triangle of C (rank-k updates) or of A (SYMM / HEMM) is referenced; Hermitian results have a real
 *      diagonal.  All run on the complex GEMM (workspaces from the library's pool). */
clblasStatus clblasCsyrk(
    clblasOrder order, clblasUplo uplo, clblasTranspose trans,
    size_t N, size_t K,
    FloatComplex alpha,
    const clblasMem A, size_t offA, size_t lda,
    FloatComplex beta,
    clblasMem C, size_t offC, size_t ldc,
    unsigned numCommandQueues, clblasQueue* commandQueues,
    unsigned numEventsInWaitList, const clblasEvent* eventWaitList, clblasEvent* events);

clblasStatus clblasZsyrk(
    clblasOrder order, clblasUplo uplo, clblasTranspose trans,
    size_t N, size_t K,
    DoubleComplex alpha,
    const clblasMem A, size_t offA, size_t lda,
    DoubleComplex beta,
    clblasMem C, size_t offC, size_t ldc,
    unsigned numCommandQueues, clblasQueue* commandQueues,
    unsigned numEventsInWaitList, const clblasEvent* eventWaitList, clblasEvent* events);

clblasStatus clblasCherk(
    clblasOrder order, clblasUplo uplo, clblasTranspose trans,
    size_t N, size_t K,
    float alpha,
    const clblasMem A, size_t offA, size_t lda,
    float beta,
    clblasMem C, size_t offC, size_t ldc,
    unsigned numCommandQueues, clblasQueue* commandQueues,
    unsigned numEventsInWaitList, const clblasEvent* eventWaitList, clblasEvent* events);

clblasStatus clblasZherk(
    clblasOrder order, clblasUplo uplo, clblasTranspose trans,
    size_t N, size_t K,
    double alpha,
    const clblasMem A, size_t offA, size_t lda,
    double beta,
    clblasMem C, size_t offC, size_t ldc,
    unsigned numCommandQueues, clblasQueue* commandQueues,
    unsigned numEventsInWaitList, const clblasEvent* eventWaitList, clblasEvent* events);

clblasStatus clblasCsyr2k(
    clblasOrder order, clblasUplo uplo, clblasTranspose trans,
    size_t N, size_t K,
    FloatComplex alpha,
    const clblasMem A, size_t offA, size_t lda,
    const clblasMem B, size_t offB, size_t ldb,
    FloatComplex beta,
    clblasMem C, size_t offC, size_t ldc,
    unsigned numCommandQueues, clblasQueue* commandQueues,
    unsigned numEventsInWaitList, const clblasEvent* eventWaitList, clblasEvent* events);

clblasStatus clblasZsyr2k(
    clblasOrder order, clblasUplo uplo, clblasTranspose trans,
    size_t N, size_t K,
    DoubleComplex alpha,
    const clblasMem A, size_t offA, size_t lda,
    const clblasMem B, size_t offB, size_t ldb,
    DoubleComplex beta,
    clblasMem C, size_t offC, size_t ldc,
    unsigned numCommandQueues, clblasQueue* commandQueues,
    unsigned numEventsInWaitList, const clblasEvent* eventWaitList, clblasEvent* events);

clblasStatus clblasCher2k(
    clblasOrder order, clblasUplo uplo, clblasTranspose trans,
    size_t N, size_t K,
    FloatComplex alpha,
    const clblasMem A, size_t offA, size_t lda,
    const clblasMem B, size_t offB, size_t ldb,
    float beta,
    clblasMem C, size_t offC, size_t ldc,
    unsigned numCommandQueues, clblasQueue* commandQueues,
    unsigned numEventsInWaitList, const clblasEvent* eventWaitList, clblasEvent* events);

clblasStatus clblasZher2k(
    clblasOrder order, clblasUplo uplo, clblasTranspose trans,
    size_t N, size_t K,
    DoubleComplex alpha,
    const clblasMem A, size_t offA, size_t lda,
    const clblasMem B, size_t offB, size_t ldb,
    double beta,
    clblasMem C, size_t offC, size_t ldc,
    unsigned numCommandQueues, clblasQueue* commandQueues,
    unsigned numEventsInWaitList, const clblasEvent* eventWaitList, clblasEvent* events);

clblasStatus clblasCsymm(
    clblasOrder order, clblasSide side, clblasUplo uplo,
    size_t M, size_t N,
    FloatComplex alpha,
    const clblasMem A, size_t offa, size_t lda,
    const clblasMem B, size_t offb, size_t ldb,
    FloatComplex beta,
    clblasMem C, size_t offc, size_t ldc,
    unsigned numCommandQueues, clblasQueue* commandQueues,
    unsigned numEventsInWaitList, const clblasEvent* eventWaitList, clblasEvent* events);

clblasStatus clblasZsymm(
    clblasOrder order, clblasSide side, clblasUplo uplo,
    size_t M, size_t N,
    DoubleComplex alpha,
    const clblasMem A, size_t offa, size_t lda,
    const clblasMem B, size_t offb, size_t ldb,
    DoubleComplex beta,
    clblasMem C, size_t offc, size_t ldc,
    unsigned numCommandQueues, clblasQueue* commandQueues,
    unsigned numEventsInWaitList, const clblasEvent* eventWaitList, clblasEvent* events);

clblasStatus clblasChemm(
    clblasOrder order, clblasSide side, clblasUplo uplo,
    size_t M, size_t N,
    FloatComplex alpha,
    const clblasMem A, size_t offa, size_t lda,
    const clblasMem B, size_t offb, size_t ldb,
    FloatComplex beta,
    clblasMem C, size_t offc, size_t ldc,
    unsigned numCommandQueues, clblasQueue* commandQueues,
    unsigned numEventsInWaitList, const clblasEvent* eventWaitList, clblasEvent* events);

clblasStatus clblasZhemm(
    clblasOrder order, clblasSide side, clblasUplo uplo,
    size_t M, size_t N,
    DoubleComplex alpha,
    const clblasMem A, size_t offa, size_t lda,
    const clblasMem B, size_t offb, size_t ldb,
    DoubleComplex beta,
    clblasMem C, size_t offc, size_t ldc,
    unsigned numCommandQueues, clblasQueue* commandQueues,
    unsigned numEventsInWaitList, const clblasEvent* eventWaitList, clblasEvent* events);

/* ---- GEMM on HOST matrices (no single counterpart in the reference: it is what a clBLAS program does with
 *      clEnqueueWriteBuffer x3 + clblasXgemm + clEnqueueReadBuffer, src/samples/example_sgemm.c:118-160, done as one
 *      call).  Same argument list as clblasSgemm / clblasDgemm, but A, B and C are HOST pointers (pinned memory for
 *      asynchronous copies; pageable memory works, staged by the driver).  Uploads, products and downloads overlap:
 *      the problem is cut into column blocks of C and K-slabs that travel and multiply in a pipeline on the
 *      library's own streams.  The work starts after what commandQueues[0] holds and the wait list; the result is
 *      in host C once commandQueues[0] (or events[0]) has completed.  Same checks and status codes as the device
 *      routines, without the memory-extent checks.  Device memory for the three matrices comes from the
 *      library's pool (clblasOutOfResources when they do not fit). */
clblasStatus clblasB200SgemmHost(
    clblasOrder order, clblasTranspose transA, clblasTranspose transB,
    size_t M, size_t N, size_t K,
    float alpha,
    const void* A, size_t offA, size_t lda,
    const void* B, size_t offB, size_t ldb,
    float beta,
    void* C, size_t offC, size_t ldc,
    unsigned numCommandQueues, clblasQueue* commandQueues,
    unsigned numEventsInWaitList, const clblasEvent* eventWaitList, clblasEvent* events);

clblasStatus clblasB200DgemmHost(
    clblasOrder order, clblasTranspose transA, clblasTranspose transB,
    size_t M, size_t N, size_t K,
    double alpha,
    const void* A, size_t offA, size_t lda,
    const void* B, size_t offB, size_t ldb,
    double beta,
    void* C, size_t offC, size_t ldc,
    unsigned numCommandQueues, clblasQueue* commandQueues,
    unsigned numEventsInWaitList, const clblasEvent* eventWaitList, clblasEvent* events);

/* ---- TRSM on HOST matrices: the argument list of clblasStrsm / clblasDtrsm with host pointers, in the manner of
 *      clblasB200SgemmHost.  The referenced triangle of A is uploaded once; B travels in blocks of independent
 *      right-hand sides (columns for clblasLeft, rows for clblasRight) that are uploaded, solved and downloaded in a
 *      pipeline.  Needs clblasSetup(), like clblasDtrsm. */
clblasStatus clblasB200StrsmHost(
    clblasOrder order, clblasSide side, clblasUplo uplo, clblasTranspose transA, clblasDiag diag,
    size_t M, size_t N,
    float alpha,
    const void* A, size_t offA, size_t lda,
    void* B, size_t offB, size_t ldb,
    unsigned numCommandQueues, clblasQueue* commandQueues,
    unsigned numEventsInWaitList, const clblasEvent* eventWaitList, clblasEvent* events);

clblasStatus clblasB200DtrsmHost(
    clblasOrder order, clblasSide side, clblasUplo uplo, clblasTranspose transA, clblasDiag diag,
    size_t M, size_t N,
    double alpha,
    const void* A, size_t offA, size_t lda,
    void* B, size_t offB, size_t ldb,
    unsigned numCommandQueues, clblasQueue* commandQueues,
    unsigned numEventsInWaitList, const clblasEvent* eventWaitList, clblasEvent* events);

/* ---- matrix helpers: replace clblasMatrixSizeInfo, clblasCreateMatrix*, clblas{Write,Read,Copy}{Sub,}Matrix{,Async}
 *      and clblasFill{Vector,SubMatrix,Matrix}{,Async} (src/clBLAS.h:9665-10238; src/library/blas/matrix.c, fill.cc).
 *      Same argument lists; `command_queue` is ONE cudaStream_t; host pointers are plain host memory (pinned memory
 *      makes the Async variants truly asynchronous).  Offsets, leading dimensions, positions and extents count
 *      elements of `element_size` bytes; for clblasRowMajor x / y and rows / columns are exchanged, as in the
 *      reference.  A region outside either matrix is clblasInvalidValue.  The blocking variants return after the
 *      stream has finished the copy; the Async variants record *event (created by the caller; may be NULL).
 *      clblasCreateMatrix* ignore `context` (the current CUDA device is used) and return cudaMalloc memory that
 *      the caller frees with cudaFree. */
clblasStatus clblasMatrixSizeInfo(clblasOrder order, size_t rows, size_t columns, size_t elemsize, size_t padding,
                                  size_t* ld, size_t* fullsize);
clblasMem clblasCreateMatrix(void* context, clblasOrder order, size_t rows, size_t columns, size_t elemsize, size_t padding,
                             size_t* ld, size_t* fullsize, int* err);
clblasMem clblasCreateMatrixWithLd(void* context, clblasOrder order, size_t rows, size_t columns, size_t elemsize, size_t ld,
                                   size_t* fullsize, int* err);
clblasMem clblasCreateMatrixFromHost(void* context, clblasOrder order, size_t rows, size_t columns, size_t elemsize, size_t ld,
                                     void* host, size_t off_host, size_t ld_host, clblasQueue command_queue,
                                     unsigned numEventsInWaitList, const clblasEvent* eventWaitList, int* err);

clblasStatus clblasWriteSubMatrix(clblasOrder order, size_t element_size, const void* A, size_t offA, size_t ldA, size_t nrA,
                                  size_t ncA, size_t xA, size_t yA, clblasMem B, size_t offB, size_t ldB, size_t nrB, size_t ncB,
                                  size_t xB, size_t yB, size_t nx, size_t ny, clblasQueue command_queue,
                                  unsigned numEventsInWaitList, const clblasEvent* eventWaitList);
clblasStatus clblasWriteSubMatrixAsync(clblasOrder order, size_t element_size, const void* A, size_t offA, size_t ldA, size_t nrA,
                                       size_t ncA, size_t xA, size_t yA, clblasMem B, size_t offB, size_t ldB, size_t nrB,
                                       size_t ncB, size_t xB, size_t yB, size_t nx, size_t ny, clblasQueue command_queue,
                                       unsigned numEventsInWaitList, const clblasEvent* eventWaitList, clblasEvent* event);
clblasStatus clblasReadSubMatrix(clblasOrder order, size_t element_size, const clblasMem A, size_t offA, size_t ldA, size_t nrA,
                                 size_t ncA, size_t xA, size_t yA, void* B, size_t offB, size_t ldB, size_t nrB, size_t ncB,
                                 size_t xB, size_t yB, size_t nx, size_t ny, clblasQueue command_queue,
                                 unsigned numEventsInWaitList, const clblasEvent* eventWaitList);
clblasStatus clblasReadSubMatrixAsync(clblasOrder order, size_t element_size, const clblasMem A, size_t offA, size_t ldA, size_t nrA,
                                      size_t ncA, size_t xA, size_t yA, void* B, size_t offB, size_t ldB, size_t nrB, size_t ncB,
                                      size_t xB, size_t yB, size_t nx, size_t ny, clblasQueue command_queue,
                                      unsigned numEventsInWaitList, const clblasEvent* eventWaitList, clblasEvent* event);
clblasStatus clblasCopySubMatrix(clblasOrder order, size_t element_size, const clblasMem A, size_t offA, size_t ldA, size_t nrA,
                                 size_t ncA, size_t xA, size_t yA, clblasMem B, size_t offB, size_t ldB, size_t nrB, size_t ncB,
                                 size_t xB, size_t yB, size_t nx, size_t ny, clblasQueue command_queue,
                                 unsigned numEventsInWaitList, const clblasEvent* eventWaitList);
clblasStatus clblasCopySubMatrixAsync(clblasOrder order, size_t element_size, const clblasMem A, size_t offA, size_t ldA, size_t nrA,
                                      size_t ncA, size_t xA, size_t yA, clblasMem B, size_t offB, size_t ldB, size_t nrB, size_t ncB,
                                      size_t xB, size_t yB, size_t nx, size_t ny, clblasQueue command_queue,
                                      unsigned numEventsInWaitList, const clblasEvent* eventWaitList, clblasEvent* event);

clblasStatus clblasWriteMatrix(clblasOrder order, size_t sx, size_t sy, size_t element_size, const void* A, size_t offA, size_t ldA,
                               clblasMem B, size_t offB, size_t ldB, clblasQueue command_queue, unsigned numEventsInWaitList,
                               const clblasEvent* eventWaitList);
clblasStatus clblasWriteMatrixAsync(clblasOrder order, size_t sx, size_t sy, size_t element_size, const void* A, size_t offA,
                                    size_t ldA, clblasMem B, size_t offB, size_t ldB, clblasQueue command_queue,
                                    unsigned numEventsInWaitList, const clblasEvent* eventWaitList, clblasEvent* event);
clblasStatus clblasReadMatrix(clblasOrder order, size_t sx, size_t sy, size_t element_size, const clblasMem A, size_t offA, size_t ldA,
                              void* B, size_t offB, size_t ldB, clblasQueue command_queue, unsigned numEventsInWaitList,
                              const clblasEvent* eventWaitList);
clblasStatus clblasReadMatrixAsync(clblasOrder order, size_t sx, size_t sy, size_t element_size, const clblasMem A, size_t offA,
                                   size_t ldA, void* B, size_t offB, size_t ldB, clblasQueue command_queue,
                                   unsigned numEventsInWaitList, const clblasEvent* eventWaitList, clblasEvent* event);
clblasStatus clblasCopyMatrix(clblasOrder order, size_t sx, size_t sy, size_t element_size, const clblasMem A, size_t offA, size_t ldA,
                              clblasMem B, size_t offB, size_t ldB, clblasQueue command_queue, unsigned numEventsInWaitList,
                              const clblasEvent* eventWaitList);
clblasStatus clblasCopyMatrixAsync(clblasOrder order, size_t sx, size_t sy, size_t element_size, const clblasMem A, size_t offA,
                                   size_t ldA, clblasMem B, size_t offB, size_t ldB, clblasQueue command_queue,
                                   unsigned numEventsInWaitList, const clblasEvent* eventWaitList, clblasEvent* event);

clblasStatus clblasFillVector(size_t nb_elem, size_t element_size, clblasMem A, size_t offA, const void* pattern,
                              clblasQueue command_queue, unsigned numEventsInWaitList, const clblasEvent* eventWaitList);
clblasStatus clblasFillVectorAsync(size_t nb_elem, size_t element_size, clblasMem A, size_t offA, const void* pattern,
                                   clblasQueue command_queue, unsigned numEventsInWaitList, const clblasEvent* eventWaitList,
                                   clblasEvent* event);
clblasStatus clblasFillSubMatrix(clblasOrder order, size_t element_size, clblasMem A, size_t offA, size_t ldA, size_t nrA,
                                 size_t ncA, size_t xA, size_t yA, size_t nx, size_t ny, const void* pattern,
                                 clblasQueue command_queue, unsigned numEventsInWaitList, const clblasEvent* eventWaitList);
clblasStatus clblasFillSubMatrixAsync(clblasOrder order, size_t element_size, clblasMem A, size_t offA, size_t ldA, size_t nrA,
                                      size_t ncA, size_t xA, size_t yA, size_t nx, size_t ny, const void* pattern,
                                      clblasQueue command_queue, unsigned numEventsInWaitList, const clblasEvent* eventWaitList,
                                      clblasEvent* event);
clblasStatus clblasFillMatrix(clblasOrder order, size_t element_size, clblasMem A, size_t offA, size_t ldA, size_t nrA, size_t ncA,
                              const void* pattern, clblasQueue command_queue, unsigned numEventsInWaitList,
                              const clblasEvent* eventWaitList);
clblasStatus clblasFillMatrixAsync(clblasOrder order, size_t element_size, clblasMem A, size_t offA, size_t ldA, size_t nrA,
                                   size_t ncA, const void* pattern, clblasQueue command_queue, unsigned numEventsInWaitList,
                                   const clblasEvent* eventWaitList, clblasEvent* event);

#ifdef __cplusplus
}
#endif
#endif /* CLBLAS_B200_H_ */
