/*
 * oracle_blas.c -- TEST INFRASTRUCTURE ONLY.  CPU restatement of the reference's own CPU BLAS
 * for the level-3 hot path (GEMM and TRSM, float and double).
 *
 * It restates NaiveBlas::gemm (src/library/tools/ktest/naive/naive_blas.cpp:546-578) and
 * NaiveBlas::trsm (:632-690) together with the index mapping of MatrixAccessor (:487-543):
 * the same loop nests, the same order of floating point operations (so results are bit-identical
 * to the reference code compiled without FMA contraction), written as plain C over raw pointers.
 * Parity is pinned: tests/test_oracle.py checks this file against the reference's own
 * naive_blas.cpp compiled from where it lies (oracle/_ref), against the reference's known-answer
 * TRSM test (src/tests/correctness/corr-trsm.cpp:240-452) and against committed golden vectors.
 *
 * Nothing in the product (clblas_b200/, include/) may call into this file; only tests/, the
 * smoke check and the benchmark's CPU-baseline leg do.
 *
 * Rows of the result are independent, so the outer loop may be split over OpenMP threads
 * without changing a single bit of the output.
 */
#include <stddef.h>

enum { ORowMajor = 0, OColumnMajor = 1 };           /* clblasOrder      */
enum { ONoTrans = 0, OTrans = 1, OConjTrans = 2 };   /* clblasTranspose  */
enum { OUpper = 0, OLower = 1 };                     /* clblasUplo       */
enum { OUnit = 0, ONonUnit = 1 };                    /* clblasDiag       */
enum { OLeft = 0, ORight = 1 };                      /* clblasSide       */

/* MatrixAccessor (naive_blas.cpp:487-543): logical (row, col) -> physical index.
 * "tra" is true when logical rows are contiguous in memory steps of 1 (column-major, no
 * transposition, or row-major with transposition). */
typedef struct { size_t ld; int tra; } acc_t;

static acc_t make_acc(int order, int trans, size_t ld)
{
    acc_t a;
    a.ld = ld;
    a.tra = ((order == OColumnMajor && trans == ONoTrans) ||
             (order == ORowMajor && trans != ONoTrans));
    return a;
}

static size_t at(acc_t a, size_t row, size_t col)
{
    return a.tra ? (row + col * a.ld) : (row * a.ld + col);
}

#define DEFINE_GEMM(NAME, T)                                                                   \
void NAME(int order, int transA, int transB, size_t M, size_t N, size_t K, T alpha,            \
          const T* A, size_t lda, const T* B, size_t ldb, T beta, T* C, size_t ldc)            \
{                                                                                              \
    acc_t ma = make_acc(order, transA, lda);                                                   \
    acc_t mb = make_acc(order, transB, ldb);                                                   \
    acc_t mc = make_acc(order, ONoTrans, ldc);                                                 \
    long long i;                                                                               \
    _Pragma("omp parallel for schedule(static)")                                               \
    for (i = 0; i < (long long)M; i++) {                                                       \
        size_t j, k;                                                                           \
        for (j = 0; j < N; j++) {                                                              \
            T tmp = (T)0.0;                                                                    \
            for (k = 0; k < K; k++) {                                                          \
                tmp = tmp + A[at(ma, (size_t)i, k)] * B[at(mb, k, j)];                         \
            }                                                                                  \
            C[at(mc, (size_t)i, j)] = C[at(mc, (size_t)i, j)] * beta + tmp * alpha;            \
        }                                                                                      \
    }                                                                                          \
}

DEFINE_GEMM(oracle_sgemm, float)
DEFINE_GEMM(oracle_dgemm, double)

/* NaiveBlas::trsm (naive_blas.cpp:632-690).  side == Right is handled, as there, by flipping
 * both accessors (solving the transposed system) and reversing the pass direction.  The solve
 * runs row by row of the (possibly flipped) system; within a row the right-hand-side columns
 * are independent, so the j loop is the one split over threads. */
#define DEFINE_TRSM(NAME, T)                                                                   \
void NAME(int order, int side, int uplo, int transA, int diag, size_t M, size_t N, T alpha,    \
          const T* A, size_t lda, T* B, size_t ldb)                                            \
{                                                                                              \
    size_t rowsA = (side == OLeft) ? M : N;                                                    \
    size_t colsB = (side == OLeft) ? N : M;                                                    \
    acc_t ma = make_acc(order, transA, lda);                                                   \
    acc_t mb = make_acc(order, ONoTrans, ldb);                                                 \
    int revPass = (uplo == OUpper) ^ (transA != ONoTrans);                                     \
    size_t i;                                                                                  \
    if (side == ORight) {                                                                      \
        ma.tra = !ma.tra;                                                                      \
        mb.tra = !mb.tra;                                                                      \
        revPass = !revPass;                                                                    \
    }                                                                                          \
    for (i = 0; i < rowsA; i++) {                                                              \
        size_t row = revPass ? (rowsA - i - 1) : i;                                            \
        size_t boundK = revPass ? (rowsA - row - 1) : row;                                     \
        long long j;                                                                           \
        _Pragma("omp parallel for schedule(static)")                                           \
        for (j = 0; j < (long long)colsB; j++) {                                               \
            T tmp = (T)0.0;                                                                    \
            size_t k;                                                                          \
            for (k = 0; k <= boundK; k++) {                                                    \
                size_t col = revPass ? (rowsA - k - 1) : k;                                    \
                if (col == row) {                                                              \
                    T a = (diag == OUnit) ? (T)1.0 : A[at(ma, row, col)];                      \
                    tmp = (B[at(mb, row, (size_t)j)] - tmp) / a;                               \
                } else {                                                                       \
                    tmp = tmp + A[at(ma, row, col)] * B[at(mb, col, (size_t)j)];               \
                }                                                                              \
            }                                                                                  \
            B[at(mb, row, (size_t)j)] = tmp;                                                   \
        }                                                                                      \
    }                                                                                          \
    for (i = 0; i < rowsA; i++) {                                                              \
        size_t j;                                                                              \
        for (j = 0; j < colsB; j++) {                                                          \
            B[at(mb, i, j)] = B[at(mb, i, j)] * alpha;                                         \
        }                                                                                      \
    }                                                                                          \
}

DEFINE_TRSM(oracle_strsm, float)
DEFINE_TRSM(oracle_dtrsm, double)

/* NaiveBlas::trmm (naive_blas.cpp:580-630): B <- alpha*op(A)*B (Left) / alpha*B*op(A) (Right), in place.
 * Rows of the (possibly flipped) system are produced in the order that only consumes values of B
 * not yet overwritten; the columns of a row are independent. */
#define DEFINE_TRMM(NAME, T)                                                                   \
void NAME(int order, int side, int uplo, int transA, int diag, size_t M, size_t N, T alpha,    \
          const T* A, size_t lda, T* B, size_t ldb)                                            \
{                                                                                              \
    size_t rowsA = (side == OLeft) ? M : N;                                                    \
    size_t colsB = (side == OLeft) ? N : M;                                                    \
    acc_t ma = make_acc(order, transA, lda);                                                   \
    acc_t mb = make_acc(order, ONoTrans, ldb);                                                 \
    int revPass = (uplo == OLower) ^ (transA != ONoTrans);                                     \
    size_t i;                                                                                  \
    if (side == ORight) {                                                                      \
        ma.tra = !ma.tra;                                                                      \
        mb.tra = !mb.tra;                                                                      \
        revPass = !revPass;                                                                    \
    }                                                                                          \
    for (i = 0; i < rowsA; i++) {                                                              \
        size_t row = revPass ? (rowsA - i - 1) : i;                                            \
        size_t boundK = revPass ? row : (rowsA - row - 1);                                     \
        long long j;                                                                           \
        _Pragma("omp parallel for schedule(static)")                                           \
        for (j = 0; j < (long long)colsB; j++) {                                               \
            T tmp = (T)0.0;                                                                    \
            size_t k;                                                                          \
            for (k = 0; k <= boundK; k++) {                                                    \
                size_t col = revPass ? k : (rowsA - k - 1);                                    \
                T a = ((k == boundK) && (diag == OUnit)) ? (T)1.0 : A[at(ma, row, col)];       \
                tmp = tmp + a * B[at(mb, col, (size_t)j)];                                     \
            }                                                                                  \
            B[at(mb, row, (size_t)j)] = tmp * alpha;                                           \
        }                                                                                      \
    }                                                                                          \
}

DEFINE_TRMM(oracle_strmm, float)
DEFINE_TRMM(oracle_dtrmm, double)

/* NaiveBlas::syrk (naive_blas.cpp:692-727): C <- alpha*op(A)*op(A)^T + beta*C on the uplo triangle of C;
 * op(A) is N x K (ConjTrans counts as Trans).  Entries outside the triangle are not touched. */
#define DEFINE_SYRK(NAME, T)                                                                   \
void NAME(int order, int uplo, int trans, size_t N, size_t K, T alpha, const T* A, size_t lda, \
          T beta, T* C, size_t ldc)                                                            \
{                                                                                              \
    acc_t ma = make_acc(order, trans == ONoTrans ? ONoTrans : OTrans, lda);                    \
    acc_t mc = make_acc(order, ONoTrans, ldc);                                                 \
    long long i;                                                                               \
    _Pragma("omp parallel for schedule(dynamic, 8)")                                           \
    for (i = 0; i < (long long)N; i++) {                                                       \
        size_t j, k;                                                                           \
        for (j = 0; j < N; j++) {                                                              \
            T tmp = (T)0.0;                                                                    \
            if ((uplo == OLower && j > (size_t)i) || (uplo == OUpper && (size_t)i > j)) continue; \
            for (k = 0; k < K; k++) {                                                          \
                tmp = tmp + A[at(ma, (size_t)i, k)] * A[at(ma, j, k)];                         \
            }                                                                                  \
            C[at(mc, (size_t)i, j)] = C[at(mc, (size_t)i, j)] * beta + tmp * alpha;            \
        }                                                                                      \
    }                                                                                          \
}

DEFINE_SYRK(oracle_ssyrk, float)
DEFINE_SYRK(oracle_dsyrk, double)

/* NaiveBlas::syr2k (naive_blas.cpp:728-766): C <- alpha*(op(A)*op(B)^T + op(B)*op(A)^T) + beta*C on the uplo
 * triangle; one running sum takes both products of each k. */
#define DEFINE_SYR2K(NAME, T)                                                                  \
void NAME(int order, int uplo, int trans, size_t N, size_t K, T alpha, const T* A, size_t lda, \
          const T* B, size_t ldb, T beta, T* C, size_t ldc)                                    \
{                                                                                              \
    int tr = trans == ONoTrans ? ONoTrans : OTrans;                                            \
    acc_t ma = make_acc(order, tr, lda);                                                       \
    acc_t mb = make_acc(order, tr, ldb);                                                       \
    acc_t mc = make_acc(order, ONoTrans, ldc);                                                 \
    long long i;                                                                               \
    _Pragma("omp parallel for schedule(dynamic, 8)")                                           \
    for (i = 0; i < (long long)N; i++) {                                                       \
        size_t j, k;                                                                           \
        for (j = 0; j < N; j++) {                                                              \
            T tmp = (T)0.0;                                                                    \
            if ((uplo == OLower && j > (size_t)i) || (uplo == OUpper && (size_t)i > j)) continue; \
            for (k = 0; k < K; k++) {                                                          \
                tmp = tmp + A[at(ma, (size_t)i, k)] * B[at(mb, j, k)] + A[at(ma, j, k)] * B[at(mb, (size_t)i, k)]; \
            }                                                                                  \
            C[at(mc, (size_t)i, j)] = C[at(mc, (size_t)i, j)] * beta + tmp * alpha;            \
        }                                                                                      \
    }                                                                                          \
}

DEFINE_SYR2K(oracle_ssyr2k, float)
DEFINE_SYR2K(oracle_dsyr2k, double)

/* SYMM.  The reference's naive BLAS has no symm; its correctness tests call the external Fortran BLAS
 * (src/tests/correctness/corr-symm.cpp -> src/tests/blas.c -> ssymm_/dsymm_, blas-lapack.h).  This is the
 * Netlib definition written in the style of NaiveBlas::gemm: C <- alpha*A*B + beta*C (Left) or
 * alpha*B*A + beta*C (Right) with A(i,j) taken from the stored uplo triangle. */
#define DEFINE_SYMM(NAME, T)                                                                   \
void NAME(int order, int side, int uplo, size_t M, size_t N, T alpha, const T* A, size_t lda,  \
          const T* B, size_t ldb, T beta, T* C, size_t ldc)                                    \
{                                                                                              \
    acc_t ma = make_acc(order, ONoTrans, lda);                                                 \
    acc_t mb = make_acc(order, ONoTrans, ldb);                                                 \
    acc_t mc = make_acc(order, ONoTrans, ldc);                                                 \
    long long i;                                                                               \
    _Pragma("omp parallel for schedule(dynamic, 8)")                                           \
    for (i = 0; i < (long long)M; i++) {                                                       \
        size_t j, k;                                                                           \
        for (j = 0; j < N; j++) {                                                              \
            T tmp = (T)0.0;                                                                    \
            if (side == OLeft) {                                                               \
                for (k = 0; k < M; k++) {                                                      \
                    int st = (uplo == OLower) ? ((size_t)i >= k) : ((size_t)i <= k);           \
                    T a = st ? A[at(ma, (size_t)i, k)] : A[at(ma, k, (size_t)i)];              \
                    tmp = tmp + a * B[at(mb, k, j)];                                           \
                }                                                                              \
            } else {                                                                           \
                for (k = 0; k < N; k++) {                                                      \
                    int st = (uplo == OLower) ? (k >= j) : (k <= j);                           \
                    T a = st ? A[at(ma, k, j)] : A[at(ma, j, k)];                              \
                    tmp = tmp + B[at(mb, (size_t)i, k)] * a;                                   \
                }                                                                              \
            }                                                                                  \
            C[at(mc, (size_t)i, j)] = C[at(mc, (size_t)i, j)] * beta + tmp * alpha;            \
        }                                                                                      \
    }                                                                                          \
}

DEFINE_SYMM(oracle_ssymm, float)
DEFINE_SYMM(oracle_dsymm, double)

/* Complex GEMM: NaiveBlas::gemm<FloatComplex / DoubleComplex> (naive_blas.cpp:546-578) with the complex
 * operators of naive_blas.cpp:297-372 written out: (a*b) = (ar*br - ai*bi, ar*bi + br*ai); an element read
 * through a ConjTrans accessor is conjugated (VectorAccessor, naive_blas.cpp:430-485).  Matrices are
 * interleaved (re, im); alpha and beta arrive as two scalars each. */
#define DEFINE_CGEMM(NAME, T)                                                                  \
void NAME(int order, int transA, int transB, size_t M, size_t N, size_t K, T alr, T ali,       \
          const T* A, size_t lda, const T* B, size_t ldb, T ber, T bei, T* C, size_t ldc)      \
{                                                                                              \
    acc_t ma = make_acc(order, transA, lda);                                                   \
    acc_t mb = make_acc(order, transB, ldb);                                                   \
    acc_t mc = make_acc(order, ONoTrans, ldc);                                                 \
    const int ca = (transA == OConjTrans), cb = (transB == OConjTrans);                        \
    long long i;                                                                               \
    _Pragma("omp parallel for schedule(static)")                                               \
    for (i = 0; i < (long long)M; i++) {                                                       \
        size_t j, k;                                                                           \
        for (j = 0; j < N; j++) {                                                              \
            T tr = (T)0.0, ti = (T)0.0;                                                        \
            for (k = 0; k < K; k++) {                                                          \
                const T* a = A + 2 * at(ma, (size_t)i, k);                                     \
                const T* b = B + 2 * at(mb, k, j);                                             \
                const T ar = a[0], ai = ca ? -a[1] : a[1];                                     \
                const T br = b[0], bi = cb ? -b[1] : b[1];                                     \
                const T pr = ar * br - ai * bi, pi = ar * bi + br * ai;                        \
                tr = tr + pr;                                                                  \
                ti = ti + pi;                                                                  \
            }                                                                                  \
            {                                                                                  \
                T* c = C + 2 * at(mc, (size_t)i, j);                                           \
                const T cr = c[0], ci = c[1];                                                  \
                const T xr = cr * ber - ci * bei, xi = cr * bei + ber * ci;                    \
                const T yr = tr * alr - ti * ali, yi = tr * ali + alr * ti;                    \
                c[0] = xr + yr;                                                                \
                c[1] = xi + yi;                                                                \
            }                                                                                  \
        }                                                                                      \
    }                                                                                          \
}

DEFINE_CGEMM(oracle_cgemm, float)
DEFINE_CGEMM(oracle_zgemm, double)

/* Complex TRSM: NaiveBlas::trsm<FloatComplex / DoubleComplex> (naive_blas.cpp:632-690) with the complex
 * operators written out; division (a/b) = ((ar*br + ai*bi)/d, (br*ai - ar*bi)/d), d = br*br + bi*bi
 * (naive_blas.cpp:333-341).  A ConjTrans accessor conjugates what it reads, also after the Right-side flip. */
#define DEFINE_CTRSM(NAME, T)                                                                  \
void NAME(int order, int side, int uplo, int transA, int diag, size_t M, size_t N, T alr, T ali, \
          const T* A, size_t lda, T* B, size_t ldb)                                            \
{                                                                                              \
    size_t rowsA = (side == OLeft) ? M : N;                                                    \
    size_t colsB = (side == OLeft) ? N : M;                                                    \
    acc_t ma = make_acc(order, transA, lda);                                                   \
    acc_t mb = make_acc(order, ONoTrans, ldb);                                                 \
    const int cj = (transA == OConjTrans);                                                     \
    int revPass = (uplo == OUpper) ^ (transA != ONoTrans);                                     \
    size_t i;                                                                                  \
    if (side == ORight) {                                                                      \
        ma.tra = !ma.tra;                                                                      \
        mb.tra = !mb.tra;                                                                      \
        revPass = !revPass;                                                                    \
    }                                                                                          \
    for (i = 0; i < rowsA; i++) {                                                              \
        size_t row = revPass ? (rowsA - i - 1) : i;                                            \
        size_t boundK = revPass ? (rowsA - row - 1) : row;                                     \
        long long j;                                                                           \
        _Pragma("omp parallel for schedule(static)")                                           \
        for (j = 0; j < (long long)colsB; j++) {                                               \
            T tr = (T)0.0, ti = (T)0.0;                                                        \
            size_t k;                                                                          \
            for (k = 0; k <= boundK; k++) {                                                    \
                size_t col = revPass ? (rowsA - k - 1) : k;                                    \
                if (col == row) {                                                              \
                    T ar = (T)1.0, ai = (T)0.0;                                                \
                    const T* b = B + 2 * at(mb, row, (size_t)j);                               \
                    const T nr = b[0] - tr, ni = b[1] - ti;                                    \
                    T d;                                                                       \
                    if (diag != OUnit) {                                                       \
                        const T* a = A + 2 * at(ma, row, col);                                 \
                        ar = a[0]; ai = cj ? -a[1] : a[1];                                     \
                    }                                                                          \
                    d = ar * ar + ai * ai;                                                     \
                    tr = (nr * ar + ni * ai) / d;                                              \
                    ti = (ar * ni - nr * ai) / d;                                              \
                } else {                                                                       \
                    const T* a = A + 2 * at(ma, row, col);                                     \
                    const T* b = B + 2 * at(mb, col, (size_t)j);                               \
                    const T ar = a[0], ai = cj ? -a[1] : a[1];                                 \
                    const T pr = ar * b[0] - ai * b[1], pi = ar * b[1] + b[0] * ai;            \
                    tr = tr + pr;                                                              \
                    ti = ti + pi;                                                              \
                }                                                                              \
            }                                                                                  \
            B[2 * at(mb, row, (size_t)j)] = tr;                                                \
            B[2 * at(mb, row, (size_t)j) + 1] = ti;                                            \
        }                                                                                      \
    }                                                                                          \
    for (i = 0; i < rowsA; i++) {                                                              \
        size_t j;                                                                              \
        for (j = 0; j < colsB; j++) {                                                          \
            T* b = B + 2 * at(mb, i, j);                                                       \
            const T xr = b[0] * alr - b[1] * ali, xi = b[0] * ali + alr * b[1];                \
            b[0] = xr;                                                                         \
            b[1] = xi;                                                                         \
        }                                                                                      \
    }                                                                                          \
}

DEFINE_CTRSM(oracle_ctrsm, float)
DEFINE_CTRSM(oracle_ztrsm, double)

/* Complex rank-k / rank-2k updates and symmetric / Hermitian products.
 * herm == 0: NaiveBlas::syrk / syr2k on FloatComplex / DoubleComplex (naive_blas.cpp:692-766; the accessor
 * treats ConjTrans as Trans there, so nothing is conjugated).  herm != 0 (HERK, HER2K, HEMM) and SYMM have no
 * counterpart in the reference's naive BLAS -- its tests call the external Fortran BLAS -- and follow the Netlib
 * definitions: C <- alpha*op(A)*op(A)^H + beta*C with real alpha, beta; C <- alpha*op(A)*op(B)^H +
 * conj(alpha)*op(B)*op(A)^H + beta*C with real beta; imaginary parts of the diagonal of C set to zero. */
#define DEFINE_CSYRK(NAME, T)                                                                  \
void NAME(int order, int uplo, int trans, int herm, size_t N, size_t K, T alr, T ali,          \
          const T* A, size_t lda, T ber, T bei, T* C, size_t ldc)                              \
{                                                                                              \
    acc_t ma = make_acc(order, trans == ONoTrans ? ONoTrans : OTrans, lda);                    \
    acc_t mc = make_acc(order, ONoTrans, ldc);                                                 \
    const int cj = herm && trans != ONoTrans;   /* op(A) = A^H: elements read conjugated */    \
    long long i;                                                                               \
    _Pragma("omp parallel for schedule(dynamic, 8)")                                           \
    for (i = 0; i < (long long)N; i++) {                                                       \
        size_t j, k;                                                                           \
        for (j = 0; j < N; j++) {                                                              \
            T tr = (T)0.0, ti = (T)0.0;                                                        \
            if ((uplo == OLower && j > (size_t)i) || (uplo == OUpper && (size_t)i > j)) continue; \
            for (k = 0; k < K; k++) {                                                          \
                const T* a = A + 2 * at(ma, (size_t)i, k);                                     \
                const T* b = A + 2 * at(ma, j, k);                                             \
                const T ar = a[0], ai = cj ? -a[1] : a[1];                                     \
                T br = b[0], bi = cj ? -b[1] : b[1];                                           \
                if (herm) bi = -bi;             /* times conj(op(A)[j][k]) */                  \
                tr = tr + (ar * br - ai * bi);                                                 \
                ti = ti + (ar * bi + br * ai);                                                 \
            }                                                                                  \
            {                                                                                  \
                T* c = C + 2 * at(mc, (size_t)i, j);                                           \
                const T cr = c[0], ci = c[1];                                                  \
                const T xr = cr * ber - ci * bei, xi = cr * bei + ber * ci;                    \
                const T yr = tr * alr - ti * ali, yi = tr * ali + alr * ti;                    \
                c[0] = xr + yr;                                                                \
                c[1] = (herm && (size_t)i == j) ? (T)0.0 : xi + yi;                            \
            }                                                                                  \
        }                                                                                      \
    }                                                                                          \
}

DEFINE_CSYRK(oracle_csyrk, float)
DEFINE_CSYRK(oracle_zsyrk, double)

#define DEFINE_CSYR2K(NAME, T)                                                                 \
void NAME(int order, int uplo, int trans, int herm, size_t N, size_t K, T alr, T ali,          \
          const T* A, size_t lda, const T* B, size_t ldb, T ber, T bei, T* C, size_t ldc)      \
{                                                                                              \
    int tr_ = trans == ONoTrans ? ONoTrans : OTrans;                                           \
    acc_t ma = make_acc(order, tr_, lda);                                                      \
    acc_t mb = make_acc(order, tr_, ldb);                                                      \
    acc_t mc = make_acc(order, ONoTrans, ldc);                                                 \
    const int cj = herm && trans != ONoTrans;                                                  \
    long long i;                                                                               \
    _Pragma("omp parallel for schedule(dynamic, 8)")                                           \
    for (i = 0; i < (long long)N; i++) {                                                       \
        size_t j, k;                                                                           \
        for (j = 0; j < N; j++) {                                                              \
            T tr = (T)0.0, ti = (T)0.0;                                                        \
            if ((uplo == OLower && j > (size_t)i) || (uplo == OUpper && (size_t)i > j)) continue; \
            for (k = 0; k < K; k++) {                                                          \
                const T* pa_i = A + 2 * at(ma, (size_t)i, k);                                  \
                const T* pa_j = A + 2 * at(ma, j, k);                                          \
                const T* pb_i = B + 2 * at(mb, (size_t)i, k);                                  \
                const T* pb_j = B + 2 * at(mb, j, k);                                          \
                const T air = pa_i[0], aii = cj ? -pa_i[1] : pa_i[1];                          \
                const T ajr = pa_j[0], aji = cj ? -pa_j[1] : pa_j[1];                          \
                const T bir = pb_i[0], bii = cj ? -pb_i[1] : pb_i[1];                          \
                const T bjr = pb_j[0], bji = cj ? -pb_j[1] : pb_j[1];                          \
                if (!herm) {                                                                   \
                    /* tmp + a_ik*b_jk + a_jk*b_ik, summed in that order (naive_blas.cpp:760) */ \
                    const T p1r = air * bjr - aii * bji, p1i = air * bji + bjr * aii;          \
                    const T p2r = ajr * bir - aji * bii, p2i = ajr * bii + bir * aji;          \
                    tr = tr + p1r + p2r;                                                       \
                    ti = ti + p1i + p2i;                                                       \
                } else {                                                                       \
                    /* alpha*a_ik*conj(b_jk) + conj(alpha)*b_ik*conj(a_jk) */                  \
                    const T p1r = air * bjr + aii * bji, p1i = aii * bjr - air * bji;          \
                    const T p2r = bir * ajr + bii * aji, p2i = bii * ajr - bir * aji;          \
                    tr = tr + (alr * p1r - ali * p1i) + (alr * p2r + ali * p2i);               \
                    ti = ti + (alr * p1i + ali * p1r) + (alr * p2i - ali * p2r);               \
                }                                                                              \
            }                                                                                  \
            {                                                                                  \
                T* c = C + 2 * at(mc, (size_t)i, j);                                           \
                const T cr = c[0], ci = c[1];                                                  \
                const T xr = cr * ber - ci * bei, xi = cr * bei + ber * ci;                    \
                if (!herm) {                                                                   \
                    const T yr = tr * alr - ti * ali, yi = tr * ali + alr * ti;                \
                    c[0] = xr + yr;                                                            \
                    c[1] = xi + yi;                                                            \
                } else {                                                                       \
                    c[0] = xr + tr;                                                            \
                    c[1] = ((size_t)i == j) ? (T)0.0 : xi + ti;                                \
                }                                                                              \
            }                                                                                  \
        }                                                                                      \
    }                                                                                          \
}

DEFINE_CSYR2K(oracle_csyr2k, float)
DEFINE_CSYR2K(oracle_zsyr2k, double)

#define DEFINE_CSYMM(NAME, T)                                                                  \
void NAME(int order, int side, int uplo, int herm, size_t M, size_t N, T alr, T ali,           \
          const T* A, size_t lda, const T* B, size_t ldb, T ber, T bei, T* C, size_t ldc)      \
{                                                                                              \
    acc_t ma = make_acc(order, ONoTrans, lda);                                                 \
    acc_t mb = make_acc(order, ONoTrans, ldb);                                                 \
    acc_t mc = make_acc(order, ONoTrans, ldc);                                                 \
    const size_t n = (side == OLeft) ? M : N;                                                  \
    long long i;                                                                               \
    _Pragma("omp parallel for schedule(dynamic, 8)")                                           \
    for (i = 0; i < (long long)M; i++) {                                                       \
        size_t j, k;                                                                           \
        for (j = 0; j < N; j++) {                                                              \
            T tr = (T)0.0, ti = (T)0.0;                                                        \
            for (k = 0; k < n; k++) {                                                          \
                /* full(r, c): entry (r, c) of the symmetric / Hermitian matrix from its stored triangle */ \
                const size_t r = (side == OLeft) ? (size_t)i : k, c = (side == OLeft) ? k : j; \
                const int st = (uplo == OLower) ? (r >= c) : (r <= c);                         \
                const T* a = A + 2 * (st ? at(ma, r, c) : at(ma, c, r));                       \
                const T* b = B + 2 * ((side == OLeft) ? at(mb, k, j) : at(mb, (size_t)i, k));  \
                T ar = a[0], ai = a[1];                                                        \
                if (herm) { if (!st) ai = -ai; if (r == c) ai = (T)0.0; }                      \
                tr = tr + (ar * b[0] - ai * b[1]);                                             \
                ti = ti + (ar * b[1] + b[0] * ai);                                             \
            }                                                                                  \
            {                                                                                  \
                T* c = C + 2 * at(mc, (size_t)i, j);                                           \
                const T cr = c[0], ci = c[1];                                                  \
                c[0] = (cr * ber - ci * bei) + (tr * alr - ti * ali);                          \
                c[1] = (cr * bei + ber * ci) + (tr * ali + alr * ti);                          \
            }                                                                                  \
        }                                                                                      \
    }                                                                                          \
}

DEFINE_CSYMM(oracle_csymm, float)
DEFINE_CSYMM(oracle_zsymm, double)

/* Complex TRMM: NaiveBlas::trmm<FloatComplex / DoubleComplex> (naive_blas.cpp:580-630) with the complex
 * operators written out; a ConjTrans accessor conjugates what it reads, also after the Right-side flip. */
#define DEFINE_CTRMM(NAME, T)                                                                  \
void NAME(int order, int side, int uplo, int transA, int diag, size_t M, size_t N, T alr, T ali, \
          const T* A, size_t lda, T* B, size_t ldb)                                            \
{                                                                                              \
    size_t rowsA = (side == OLeft) ? M : N;                                                    \
    size_t colsB = (side == OLeft) ? N : M;                                                    \
    acc_t ma = make_acc(order, transA, lda);                                                   \
    acc_t mb = make_acc(order, ONoTrans, ldb);                                                 \
    const int cj = (transA == OConjTrans);                                                     \
    int revPass = (uplo == OLower) ^ (transA != ONoTrans);                                     \
    size_t i;                                                                                  \
    if (side == ORight) {                                                                      \
        ma.tra = !ma.tra;                                                                      \
        mb.tra = !mb.tra;                                                                      \
        revPass = !revPass;                                                                    \
    }                                                                                          \
    for (i = 0; i < rowsA; i++) {                                                              \
        size_t row = revPass ? (rowsA - i - 1) : i;                                            \
        size_t boundK = revPass ? row : (rowsA - row - 1);                                     \
        long long j;                                                                           \
        _Pragma("omp parallel for schedule(static)")                                           \
        for (j = 0; j < (long long)colsB; j++) {                                               \
            T tr = (T)0.0, ti = (T)0.0;                                                        \
            size_t k;                                                                          \
            for (k = 0; k <= boundK; k++) {                                                    \
                size_t col = revPass ? k : (rowsA - k - 1);                                    \
                T ar = (T)1.0, ai = (T)0.0;                                                    \
                const T* b = B + 2 * at(mb, col, (size_t)j);                                   \
                if (!((k == boundK) && (diag == OUnit))) {                                     \
                    const T* a = A + 2 * at(ma, row, col);                                     \
                    ar = a[0]; ai = cj ? -a[1] : a[1];                                         \
                }                                                                              \
                tr = tr + (ar * b[0] - ai * b[1]);                                             \
                ti = ti + (ar * b[1] + b[0] * ai);                                             \
            }                                                                                  \
            B[2 * at(mb, row, (size_t)j)] = tr * alr - ti * ali;                               \
            B[2 * at(mb, row, (size_t)j) + 1] = tr * ali + alr * ti;                           \
        }                                                                                      \
    }                                                                                          \
}

DEFINE_CTRMM(oracle_ctrmm, float)
DEFINE_CTRMM(oracle_ztrmm, double)
