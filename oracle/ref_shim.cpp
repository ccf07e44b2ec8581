/*
 * ref_shim.cpp -- TEST INFRASTRUCTURE ONLY.  Builds the reference's own CPU BLAS,
 * src/library/tools/ktest/naive/naive_blas.cpp, from where it lies in the reference tree
 * (the include directory is given on the compiler command line by oracle/Makefile; no copy of
 * the reference source is kept in this repository) and exports NaiveBlas::gemm / NaiveBlas::trsm
 * for float and double with C linkage.  The output goes to oracle/_ref/libnaive_ref.so.
 *
 * naive_blas.cpp expects the OpenCL scalar and 2-vector typedefs; the few it uses are declared
 * here so that no OpenCL header is needed.
 */
#include <cstddef>
#include <cmath>
#include <string>

typedef int                cl_int;
typedef unsigned int       cl_uint;
typedef unsigned long long cl_ulong;
typedef float              cl_float;
typedef double             cl_double;
typedef struct { float s[2]; }  cl_float2;
typedef struct { double s[2]; } cl_double2;
using std::isnan;

#include "naive_blas.cpp"

extern "C" {

void ref_sgemm(int order, int transA, int transB, size_t M, size_t N, size_t K, float alpha,
               const float* A, size_t lda, const float* B, size_t ldb, float beta, float* C, size_t ldc)
{
    NaiveBlas::gemm<float>((NaiveBlas::clblasOrder)order, (NaiveBlas::clblasTranspose)transA,
                           (NaiveBlas::clblasTranspose)transB, M, N, K, alpha, A, lda, B, ldb, beta, C, ldc);
}

void ref_dgemm(int order, int transA, int transB, size_t M, size_t N, size_t K, double alpha,
               const double* A, size_t lda, const double* B, size_t ldb, double beta, double* C, size_t ldc)
{
    NaiveBlas::gemm<double>((NaiveBlas::clblasOrder)order, (NaiveBlas::clblasTranspose)transA,
                            (NaiveBlas::clblasTranspose)transB, M, N, K, alpha, A, lda, B, ldb, beta, C, ldc);
}

void ref_strsm(int order, int side, int uplo, int transA, int diag, size_t M, size_t N, float alpha,
               const float* A, size_t lda, float* B, size_t ldb)
{
    NaiveBlas::trsm<float>((NaiveBlas::clblasOrder)order, (NaiveBlas::clblasSide)side,
                           (NaiveBlas::clblasUplo)uplo, (NaiveBlas::clblasTranspose)transA,
                           (NaiveBlas::clblasDiag)diag, M, N, alpha, A, lda, B, ldb);
}

void ref_dtrsm(int order, int side, int uplo, int transA, int diag, size_t M, size_t N, double alpha,
               const double* A, size_t lda, double* B, size_t ldb)
{
    NaiveBlas::trsm<double>((NaiveBlas::clblasOrder)order, (NaiveBlas::clblasSide)side,
                            (NaiveBlas::clblasUplo)uplo, (NaiveBlas::clblasTranspose)transA,
                            (NaiveBlas::clblasDiag)diag, M, N, alpha, A, lda, B, ldb);
}

void ref_strmm(int order, int side, int uplo, int transA, int diag, size_t M, size_t N, float alpha,
               const float* A, size_t lda, float* B, size_t ldb)
{
    NaiveBlas::trmm<float>((NaiveBlas::clblasOrder)order, (NaiveBlas::clblasSide)side,
                           (NaiveBlas::clblasUplo)uplo, (NaiveBlas::clblasTranspose)transA,
                           (NaiveBlas::clblasDiag)diag, M, N, alpha, A, lda, B, ldb);
}

void ref_dtrmm(int order, int side, int uplo, int transA, int diag, size_t M, size_t N, double alpha,
               const double* A, size_t lda, double* B, size_t ldb)
{
    NaiveBlas::trmm<double>((NaiveBlas::clblasOrder)order, (NaiveBlas::clblasSide)side,
                            (NaiveBlas::clblasUplo)uplo, (NaiveBlas::clblasTranspose)transA,
                            (NaiveBlas::clblasDiag)diag, M, N, alpha, A, lda, B, ldb);
}

void ref_ssyrk(int order, int uplo, int trans, size_t N, size_t K, float alpha, const float* A, size_t lda,
               float beta, float* C, size_t ldc)
{
    NaiveBlas::syrk<float>((NaiveBlas::clblasOrder)order, (NaiveBlas::clblasUplo)uplo, (NaiveBlas::clblasTranspose)trans,
                           N, K, alpha, A, lda, beta, C, ldc);
}

void ref_dsyrk(int order, int uplo, int trans, size_t N, size_t K, double alpha, const double* A, size_t lda,
               double beta, double* C, size_t ldc)
{
    NaiveBlas::syrk<double>((NaiveBlas::clblasOrder)order, (NaiveBlas::clblasUplo)uplo, (NaiveBlas::clblasTranspose)trans,
                            N, K, alpha, A, lda, beta, C, ldc);
}

void ref_ssyr2k(int order, int uplo, int trans, size_t N, size_t K, float alpha, const float* A, size_t lda,
                const float* B, size_t ldb, float beta, float* C, size_t ldc)
{
    NaiveBlas::syr2k<float>((NaiveBlas::clblasOrder)order, (NaiveBlas::clblasUplo)uplo, (NaiveBlas::clblasTranspose)trans,
                            N, K, alpha, A, lda, B, ldb, beta, C, ldc);
}

void ref_dsyr2k(int order, int uplo, int trans, size_t N, size_t K, double alpha, const double* A, size_t lda,
                const double* B, size_t ldb, double beta, double* C, size_t ldc)
{
    NaiveBlas::syr2k<double>((NaiveBlas::clblasOrder)order, (NaiveBlas::clblasUplo)uplo, (NaiveBlas::clblasTranspose)trans,
                             N, K, alpha, A, lda, B, ldb, beta, C, ldc);
}

void ref_cgemm(int order, int transA, int transB, size_t M, size_t N, size_t K, float alr, float ali,
               const float* A, size_t lda, const float* B, size_t ldb, float ber, float bei, float* C, size_t ldc)
{
    NaiveBlas::gemm<NaiveBlas::FloatComplex>((NaiveBlas::clblasOrder)order, (NaiveBlas::clblasTranspose)transA,
                                  (NaiveBlas::clblasTranspose)transB, M, N, K, NaiveBlas::floatComplex(alr, ali),
                                  reinterpret_cast<const NaiveBlas::FloatComplex*>(A), lda, reinterpret_cast<const NaiveBlas::FloatComplex*>(B), ldb,
                                  NaiveBlas::floatComplex(ber, bei), reinterpret_cast<NaiveBlas::FloatComplex*>(C), ldc);
}

void ref_zgemm(int order, int transA, int transB, size_t M, size_t N, size_t K, double alr, double ali,
               const double* A, size_t lda, const double* B, size_t ldb, double ber, double bei, double* C, size_t ldc)
{
    NaiveBlas::gemm<NaiveBlas::DoubleComplex>((NaiveBlas::clblasOrder)order, (NaiveBlas::clblasTranspose)transA,
                                   (NaiveBlas::clblasTranspose)transB, M, N, K, NaiveBlas::doubleComplex(alr, ali),
                                   reinterpret_cast<const NaiveBlas::DoubleComplex*>(A), lda, reinterpret_cast<const NaiveBlas::DoubleComplex*>(B), ldb,
                                   NaiveBlas::doubleComplex(ber, bei), reinterpret_cast<NaiveBlas::DoubleComplex*>(C), ldc);
}

void ref_ctrsm(int order, int side, int uplo, int transA, int diag, size_t M, size_t N, float alr, float ali,
               const float* A, size_t lda, float* B, size_t ldb)
{
    NaiveBlas::trsm<NaiveBlas::FloatComplex>((NaiveBlas::clblasOrder)order, (NaiveBlas::clblasSide)side, (NaiveBlas::clblasUplo)uplo,
                                             (NaiveBlas::clblasTranspose)transA, (NaiveBlas::clblasDiag)diag, M, N,
                                             NaiveBlas::floatComplex(alr, ali), reinterpret_cast<const NaiveBlas::FloatComplex*>(A), lda,
                                             reinterpret_cast<NaiveBlas::FloatComplex*>(B), ldb);
}

void ref_ztrsm(int order, int side, int uplo, int transA, int diag, size_t M, size_t N, double alr, double ali,
               const double* A, size_t lda, double* B, size_t ldb)
{
    NaiveBlas::trsm<NaiveBlas::DoubleComplex>((NaiveBlas::clblasOrder)order, (NaiveBlas::clblasSide)side, (NaiveBlas::clblasUplo)uplo,
                                              (NaiveBlas::clblasTranspose)transA, (NaiveBlas::clblasDiag)diag, M, N,
                                              NaiveBlas::doubleComplex(alr, ali), reinterpret_cast<const NaiveBlas::DoubleComplex*>(A), lda,
                                              reinterpret_cast<NaiveBlas::DoubleComplex*>(B), ldb);
}

#define REF_CSYRK(NAME, CT, MK, T)                                                                                   \
    void NAME(int order, int uplo, int trans, size_t N, size_t K, T alr, T ali, const T* A, size_t lda, T ber, T bei,    \
              T* C, size_t ldc)                                                                                          \
    {                                                                                                                    \
        NaiveBlas::syrk<NaiveBlas::CT>((NaiveBlas::clblasOrder)order, (NaiveBlas::clblasUplo)uplo,                       \
                                       (NaiveBlas::clblasTranspose)trans, N, K, NaiveBlas::MK(alr, ali),                 \
                                       reinterpret_cast<const NaiveBlas::CT*>(A), lda, NaiveBlas::MK(ber, bei),          \
                                       reinterpret_cast<NaiveBlas::CT*>(C), ldc);                                        \
    }
REF_CSYRK(ref_csyrk, FloatComplex, floatComplex, float)
REF_CSYRK(ref_zsyrk, DoubleComplex, doubleComplex, double)

#define REF_CSYR2K(NAME, CT, MK, T)                                                                                  \
    void NAME(int order, int uplo, int trans, size_t N, size_t K, T alr, T ali, const T* A, size_t lda, const T* B,      \
              size_t ldb, T ber, T bei, T* C, size_t ldc)                                                                \
    {                                                                                                                    \
        NaiveBlas::syr2k<NaiveBlas::CT>((NaiveBlas::clblasOrder)order, (NaiveBlas::clblasUplo)uplo,                      \
                                        (NaiveBlas::clblasTranspose)trans, N, K, NaiveBlas::MK(alr, ali),                \
                                        reinterpret_cast<const NaiveBlas::CT*>(A), lda,                                  \
                                        reinterpret_cast<const NaiveBlas::CT*>(B), ldb, NaiveBlas::MK(ber, bei),         \
                                        reinterpret_cast<NaiveBlas::CT*>(C), ldc);                                       \
    }
REF_CSYR2K(ref_csyr2k, FloatComplex, floatComplex, float)
REF_CSYR2K(ref_zsyr2k, DoubleComplex, doubleComplex, double)

#define REF_CTRMM(NAME, CT, MK, T)                                                                                   \
    void NAME(int order, int side, int uplo, int transA, int diag, size_t M, size_t N, T alr, T ali, const T* A,         \
              size_t lda, T* B, size_t ldb)                                                                              \
    {                                                                                                                    \
        NaiveBlas::trmm<NaiveBlas::CT>((NaiveBlas::clblasOrder)order, (NaiveBlas::clblasSide)side,                       \
                                       (NaiveBlas::clblasUplo)uplo, (NaiveBlas::clblasTranspose)transA,                  \
                                       (NaiveBlas::clblasDiag)diag, M, N, NaiveBlas::MK(alr, ali),                       \
                                       reinterpret_cast<const NaiveBlas::CT*>(A), lda, reinterpret_cast<NaiveBlas::CT*>(B), ldb); \
    }
REF_CTRMM(ref_ctrmm, FloatComplex, floatComplex, float)
REF_CTRMM(ref_ztrmm, DoubleComplex, doubleComplex, double)

}  // extern "C"
