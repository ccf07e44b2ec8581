// Tile-config dispatcher: chooses the kernel family for one column-major GEMM from precision,
// transposes, shape and operand alignment.  It stands where the reference has the generated
// gemmSelectKernel<T> decision tree and the shape-triggered GemmSpecialCases
// (src/library/blas/AutoGemm/KernelSelection.py:30-305, src/library/blas/specialCases/
// GemmSpecialCases.cpp:827-952): the reference picks the largest tile that divides M and N and
// pays extra launches otherwise; here every family handles ragged M, N, K in one launch, so the
// only question is whether the operands can be fetched by TMA (16-byte aligned base addresses
// and leading dimensions) or need the element-granular loader.
#include "common.h"

namespace cb200 {

template <typename T>
static cudaError_t degenerate(const GemmProblem<T>& p, cudaStream_t s, bool* handled)
{
    *handled = true;
    if (p.M == 0 || p.N == 0) return cudaSuccess;
    if (p.K == 0 || p.alpha == T(0)) {
        // BLAS semantics: C <- beta*C, A and B are not referenced.
        set_last_kernel("scale");
        if (p.beta == T(1)) return cudaSuccess;
        return launch_scale<T>(p.M, p.N, p.beta, p.C, p.ldc, s);
    }
    *handled = false;
    return cudaSuccess;
}

template <>
cudaError_t gemm_colmajor<float>(const GemmProblem<float>& p, cudaStream_t s)
{
    bool handled;
    cudaError_t e = degenerate(p, s, &handled);
    if (handled) return e;
    if (forced_gemm_path() != PATH_SIMT_LDG) {
        e = launch_sgemm_ffma_tma(p, s);
        if (e != cudaErrorNotSupported) return e;
    }
    return launch_gemm_simt<float>(p, s);
}

template <>
cudaError_t gemm_colmajor<double>(const GemmProblem<double>& p, cudaStream_t s)
{
    bool handled;
    cudaError_t e = degenerate(p, s, &handled);
    if (handled) return e;
    if (forced_gemm_path() != PATH_SIMT_LDG) {
        e = launch_dgemm_mma_tma(p, s);
        if (e != cudaErrorNotSupported) return e;
    }
    return launch_gemm_simt<double>(p, s);
}

}  // namespace cb200
