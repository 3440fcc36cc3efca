// Elementwise fp16 steps between the quantized GEMMs of a decoder block, as single launches that take part in the
// programmatic-dependent-launch chain of the GEMMs around them: SiLU(gate) * up (what the reference's FasterTransformer fork
// does with genericActivation after the gate / up GEMMs, layers/FfnLayer.cc:407-421) and the residual add
// (invokeAddBiasResidual without bias).  16 bytes per thread and access; inputs are read after the dependency wait.
#include <cuda_fp16.h>

#include "abq_common.cuh"
#include "abq_kernels.h"

namespace abq {

constexpr int kGlueThreads = 256;

// out[m][f] = silu(gu[m][f]) * gu[m][F + f], f < F (F % 8 == 0)
__global__ void __launch_bounds__(kGlueThreads) swiglu_half_kernel(const __half *__restrict__ gu, __half *__restrict__ out, int M, int F)
{
    pdl_launch_dependents();
    const long idx = ((long)blockIdx.x * kGlueThreads + threadIdx.x) * 8;
    pdl_wait_prior_grid();
    if (idx >= (long)M * F)
        return;
    const long m = idx / F, f = idx - m * F;
    const uint4 g = *reinterpret_cast<const uint4 *>(gu + m * 2 * F + f);
    const uint4 u = *reinterpret_cast<const uint4 *>(gu + m * 2 * F + F + f);
    const __half2 *gh = reinterpret_cast<const __half2 *>(&g), *uh = reinterpret_cast<const __half2 *>(&u);
    uint4 o;
    __half2 *oh = reinterpret_cast<__half2 *>(&o);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        const float2 a = __half22float2(gh[e]), b = __half22float2(uh[e]);
        // silu in fp32, rounded to fp16 before the product, as two separate fp16 kernels would leave it
        const __half2 s = __floats2half2_rn(a.x / (1.f + __expf(-a.x)), a.y / (1.f + __expf(-a.y)));
        oh[e] = __hmul2(s, __floats2half2_rn(b.x, b.y));
    }
    *reinterpret_cast<uint4 *>(out + idx) = o;
}

__global__ void __launch_bounds__(kGlueThreads) add_half_kernel(const __half *__restrict__ a, const __half *__restrict__ b, __half *__restrict__ out, long n)
{
    pdl_launch_dependents();
    const long idx = ((long)blockIdx.x * kGlueThreads + threadIdx.x) * 8;
    pdl_wait_prior_grid();
    if (idx >= n)
        return;
    const uint4 x = *reinterpret_cast<const uint4 *>(a + idx), y = *reinterpret_cast<const uint4 *>(b + idx);
    const __half2 *xh = reinterpret_cast<const __half2 *>(&x), *yh = reinterpret_cast<const __half2 *>(&y);
    uint4 o;
    __half2 *oh = reinterpret_cast<__half2 *>(&o);
#pragma unroll
    for (int e = 0; e < 4; ++e)
        oh[e] = __hadd2(xh[e], yh[e]);
    *reinterpret_cast<uint4 *>(out + idx) = o;
}

template <typename Kernel, typename... Args>
static cudaError_t launch_pdl(Kernel kern, long items, cudaStream_t stream, Args... args)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)((items / 8 + kGlueThreads - 1) / kGlueThreads));
    cfg.blockDim = dim3(kGlueThreads);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kern, args...);
}

cudaError_t swiglu_half(const __half *gu, __half *out, int M, int F, cudaStream_t stream)
{
    return launch_pdl(swiglu_half_kernel, (long)M * F, stream, gu, out, M, F);
}

cudaError_t add_half(const __half *a, const __half *b, __half *out, long n, cudaStream_t stream)
{
    return launch_pdl(add_half_kernel, n, stream, a, b, out, n);
}

} // namespace abq

extern "C" abq_status abq_swiglu_half(const void *gate_up, void *out, int M, int F, abq_stream_t stream)
{
    if (!gate_up || !out || M <= 0 || F <= 0 || F % 8 != 0 || ((reinterpret_cast<uintptr_t>(gate_up) | reinterpret_cast<uintptr_t>(out)) & 15))
        return ABQ_ERR_INVALID_ARG;
    cudaError_t e = abq::swiglu_half(reinterpret_cast<const __half *>(gate_up), reinterpret_cast<__half *>(out), M, F, reinterpret_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) {
        abq::set_last_cuda_error(e);
        return ABQ_ERR_CUDA;
    }
    return ABQ_OK;
}

extern "C" abq_status abq_add_half(const void *a, const void *b, void *out, long n, abq_stream_t stream)
{
    if (!a || !b || !out || n <= 0 || n % 8 != 0 ||
        ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(out)) & 15))
        return ABQ_ERR_INVALID_ARG;
    cudaError_t e = abq::add_half(reinterpret_cast<const __half *>(a), reinterpret_cast<const __half *>(b), reinterpret_cast<__half *>(out), n,
                                  reinterpret_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) {
        abq::set_last_cuda_error(e);
        return ABQ_ERR_CUDA;
    }
    return ABQ_OK;
}
