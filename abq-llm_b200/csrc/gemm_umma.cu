// Route B placeholder while the tcgen05 kernel is being brought up.
#include "abq_kernels.h"
namespace abq {
abq_status umma_plan(abq_gemm_state *) { return ABQ_ERR_UNSUPPORTED; }
cudaError_t umma_launch(const abq_gemm_state *, cudaStream_t) { return cudaErrorNotSupported; }
size_t umma_workspace_bytes(int M, int N, int K) { return (size_t)M * K + (size_t)N * K; }
}
