#include "common.h"
namespace cb200 {
cudaError_t launch_dgemm_mma_tma(const GemmProblem<double>&, cudaStream_t) { return cudaErrorNotSupported; }
cudaError_t launch_sgemm_ffma_tma(const GemmProblem<float>&, cudaStream_t) { return cudaErrorNotSupported; }
}
