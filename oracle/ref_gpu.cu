// Test infrastructure, not part of the product: a C entry point over a few instantiations of the REFERENCE's own GPU
// kernel templates, compiled from its headers where they lie (engine/common/base.h, engine/mma_any/aq_bmma_op.h,
// aq_bmma_kernel.h, bmma.h).  Used on a GPU box to (1) pin the oracle and the product against what the reference's
// kernels really output and (2) time the reference's own kernels beside ours.  Nothing of the reference is copied:
// this file only names its public template parameters, the way its instantiation files do
// (engine/mma_any/aq_bmma_impl/*.cu through AQ_INSTANTIATE_FUN, engine/common/base.h:144-166).
//
// Configurations: the two W2A8 tiles FasterTransformer's wrapper hard-codes (abq_gemm_wrapper.cu:100-124: M == 1 and
// M > 1, signed and unsigned) and one W4A4 tile of the engine's search space (aq_bmma_impl/aq_bmma_w4a4.h:22).
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "common/base.h"
#include "mma_any/aq_bmma_op.h"

// id 0 / 1: W2A8 decode tile (M == 1), signed / unsigned
AQ_INSTANTIATE_FUN(AqBMMA, 8, 2, true, 1, 48, 512, 8, 24, 128, 8, 8, 128, 4);
AQ_INSTANTIATE_FUN(AqBMMA, 8, 2, false, 1, 48, 512, 8, 24, 128, 8, 8, 128, 4);
// id 2 / 3: W2A8 tile for M > 1, signed / unsigned
AQ_INSTANTIATE_FUN(AqBMMA, 8, 2, true, 8, 48, 256, 32, 48, 128, 8, 8, 128, 5);
AQ_INSTANTIATE_FUN(AqBMMA, 8, 2, false, 8, 48, 256, 32, 48, 128, 8, 8, 128, 5);
// id 4: W4A4 signed, cta <2,32,256>
AQ_INSTANTIATE_FUN(AqBMMA, 4, 4, true, 2, 32, 256, 8, 64, 128, 8, 8, 128, 2);

namespace {
struct Entry {
    AqBMMAInitFn_t init;
    AqBMMAExecFn_t exec;
    int x_bits, w_bits, is_signed;
};
Entry entry(int id)
{
    switch (id) {
    case 0: return { AQ_NAME_FUN(AqBMMA, Init, 8, 2, true, 1, 48, 512, 8, 24, 128, 8, 8, 128, 4),
                     AQ_NAME_FUN(AqBMMA, Exec, 8, 2, true, 1, 48, 512, 8, 24, 128, 8, 8, 128, 4), 8, 2, 1 };
    case 1: return { AQ_NAME_FUN(AqBMMA, Init, 8, 2, false, 1, 48, 512, 8, 24, 128, 8, 8, 128, 4),
                     AQ_NAME_FUN(AqBMMA, Exec, 8, 2, false, 1, 48, 512, 8, 24, 128, 8, 8, 128, 4), 8, 2, 0 };
    case 2: return { AQ_NAME_FUN(AqBMMA, Init, 8, 2, true, 8, 48, 256, 32, 48, 128, 8, 8, 128, 5),
                     AQ_NAME_FUN(AqBMMA, Exec, 8, 2, true, 8, 48, 256, 32, 48, 128, 8, 8, 128, 5), 8, 2, 1 };
    case 3: return { AQ_NAME_FUN(AqBMMA, Init, 8, 2, false, 8, 48, 256, 32, 48, 128, 8, 8, 128, 5),
                     AQ_NAME_FUN(AqBMMA, Exec, 8, 2, false, 8, 48, 256, 32, 48, 128, 8, 8, 128, 5), 8, 2, 0 };
    case 4: return { AQ_NAME_FUN(AqBMMA, Init, 4, 4, true, 2, 32, 256, 8, 64, 128, 8, 8, 128, 2),
                     AQ_NAME_FUN(AqBMMA, Exec, 4, 4, true, 2, 32, 256, 8, 64, 128, 8, 8, 128, 2), 4, 4, 1 };
    default: return { nullptr, nullptr, 0, 0, 0 };
    }
}
} // namespace

extern "C" {

// x_bits / w_bits / signedness of configuration `id`; returns 0 for an unknown id
__attribute__((visibility("default"))) int abq_ref_gpu_config(int id, int *x_bits, int *w_bits, int *is_signed)
{
    const Entry e = entry(id);
    if (!e.init)
        return 0;
    *x_bits = e.x_bits;
    *w_bits = e.w_bits;
    *is_signed = e.is_signed;
    return 1;
}

// One GEMM with the reference's kernel: X, W bit-planes, D int32 [M][N], all device pointers.  `repeats` launches
// (timing loops call it with repeats > 1).  Returns 0 on success, 1 unknown id, 2 the reference's own initialisation
// refused the shape, 3 a CUDA launch error.
__attribute__((visibility("default"))) int abq_ref_gpu_gemm(int id, int *X, int *W, int M, int N, int K, int *D, int repeats, void *stream)
{
    const Entry e = entry(id);
    if (!e.init)
        return 1;
    AqBMMAOpState st = (*e.init)(X, W, M, N, K, D, nullptr, false);
    if (!st.initSuccess)
        return 2;
    for (int i = 0; i < repeats; ++i)
        (*e.exec)(st, reinterpret_cast<cudaStream_t>(stream));
    return cudaGetLastError() == cudaSuccess ? 0 : 3;
}
}
