// Decode route over prepared weights: the kernels for 3-bit weights (a compile unit per width, so that they build in parallel).
#include "gemm_stream_kernel.cuh"

namespace abq {
ABQ_STREAM_WIDTH(3)
} // namespace abq
