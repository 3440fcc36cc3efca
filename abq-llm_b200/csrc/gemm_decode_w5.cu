// decode_kernel for 5-bit weights (all token-tile, scale-mode and warp-count variants)
#include "gemm_decode_kernel.cuh"

namespace abq {
ABQ_DECODE_WIDTH(5)
} // namespace abq
