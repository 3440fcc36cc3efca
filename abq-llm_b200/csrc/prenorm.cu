// The steps a decoder block runs between one quantized GEMM and the next, as ONE launch: (residual add) -> RMSNorm ->
// activation quantiser -> bit-planes.  In the reference's FasterTransformer fork these are separate kernels
// (invokeGeneralAddBiasResidualPreLayerNorm / invokeGeneralT5LayerNorm, then ABQGEMMWrapper::pack = pack_half,
// kernels/abqgemm/abq_gemm_wrapper.cu:79-98); every one of them reads and writes the whole activation matrix.  Here a row
// is read once, kept in registers, and leaves as planes (and, where a caller wants them, as the fp16 sum and the fp16
// normalised row, bit-identical to what the separate kernels would have written):
//     s[k]  = a[k] + b[k]                                  (fp16 add; only with a residual)
//     y[k]  = half((float(s[k]) * rsqrt(mean(s^2) + eps)) * float(gamma[k]))
//     code  = MODE 0: (int)(y * half(scale[0]))            the wrapper's quantiser: fp16 product, truncation, no clamp
//             MODE 1: clamp(rint(float(y) / scale[row]))   given per-token scales
//             MODE 2: as 1 with scale[row] = max|y| / (2^(bits-1) - 1), computed here and written to row_scale_out
// One CTA per token row, one thread per run of 32 features (two runs per thread at most: K <= 16384).
#include <cuda_fp16.h>

#include "abq_common.cuh"
#include "abq_kernels.h"

namespace abq {

constexpr int kNormThreads = 256;
constexpr int kNormRuns = 2; // runs of 32 features per thread

struct PrenormArgs {
    const __half *a, *b;  // b: residual or null
    __half *sum_out;      // a + b, or null
    const __half *gamma;
    float eps;
    const float *scale;   // MODE 0: one value; MODE 1: per row; MODE 2: unused
    float *row_scale_out; // MODE 2: per row
    uint32_t *planes;     // [bits][rows][K/32] or null
    __half *y_out;        // normalised row or null
    int rows, K;
};

__device__ __forceinline__ float block_reduce(float v, bool take_max, float *scratch)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float u = __shfl_xor_sync(0xffffffffu, v, o);
        v = take_max ? fmaxf(v, u) : v + u;
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads(); // scratch may still be read from the previous reduction
    if (lane == 0)
        scratch[warp] = v;
    __syncthreads();
    float r = scratch[0];
#pragma unroll
    for (int w = 1; w < kNormThreads / 32; ++w)
        r = take_max ? fmaxf(r, scratch[w]) : r + scratch[w]; // the same order in every thread
    return r;
}

template <int BITS, int MODE>
__global__ void __launch_bounds__(kNormThreads) rmsnorm_quantize_pack_kernel(const PrenormArgs p)
{
    __shared__ float scratch[kNormThreads / 32];
    pdl_launch_dependents();
    const int row = blockIdx.x;
    const int kw = p.K >> 5;
    const long L = (long)p.rows * kw;
    uint4 v[kNormRuns][4];
    uint4 gm[kNormRuns][4];
    // gamma does not depend on the kernel launched before: fetch it ahead of the dependency wait
#pragma unroll
    for (int r = 0; r < kNormRuns; ++r) {
        const int run = threadIdx.x + r * kNormThreads;
        if (run < kw) {
#pragma unroll
            for (int i = 0; i < 4; ++i)
                gm[r][i] = __ldg(reinterpret_cast<const uint4 *>(p.gamma + (size_t)run * 32) + i);
        }
    }
    pdl_wait_prior_grid();
    float ss = 0.f;
#pragma unroll
    for (int r = 0; r < kNormRuns; ++r) {
        const int run = threadIdx.x + r * kNormThreads;
        if (run < kw) {
            const size_t at = (size_t)row * p.K + (size_t)run * 32;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                v[r][i] = *(reinterpret_cast<const uint4 *>(p.a + at) + i);
                if (p.b) {
                    const uint4 o = *(reinterpret_cast<const uint4 *>(p.b + at) + i);
                    __half2 *x = reinterpret_cast<__half2 *>(&v[r][i]);
                    const __half2 *y = reinterpret_cast<const __half2 *>(&o);
#pragma unroll
                    for (int e = 0; e < 4; ++e)
                        x[e] = __hadd2(x[e], y[e]);
                    if (p.sum_out)
                        *(reinterpret_cast<uint4 *>(p.sum_out + at) + i) = v[r][i];
                }
                const __half2 *x = reinterpret_cast<const __half2 *>(&v[r][i]);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float2 f = __half22float2(x[e]);
                    ss = fmaf(f.x, f.x, ss);
                    ss = fmaf(f.y, f.y, ss);
                }
            }
        }
    }
    ss = block_reduce(ss, false, scratch);
    const float rs = __frsqrt_rn(__fadd_rn(__fdiv_rn(ss, (float)p.K), p.eps));
    // normalise in place
    float amax = 0.f;
#pragma unroll
    for (int r = 0; r < kNormRuns; ++r) {
        const int run = threadIdx.x + r * kNormThreads;
        if (run < kw) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                __half2 *x = reinterpret_cast<__half2 *>(&v[r][i]);
                const __half2 *gh = reinterpret_cast<const __half2 *>(&gm[r][i]);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float2 f = __half22float2(x[e]), gf = __half22float2(gh[e]);
                    x[e] = __floats2half2_rn(__fmul_rn(__fmul_rn(f.x, rs), gf.x), __fmul_rn(__fmul_rn(f.y, rs), gf.y));
                    if (MODE == 2) {
                        const float2 y = __half22float2(x[e]);
                        amax = fmaxf(amax, fmaxf(fabsf(y.x), fabsf(y.y)));
                    }
                }
                if (p.y_out)
                    *(reinterpret_cast<uint4 *>(p.y_out + (size_t)row * p.K + (size_t)run * 32) + i) = v[r][i];
            }
        }
    }
    if (!p.planes)
        return;
    const int qmin = -(1 << (BITS - 1)), qmax = (1 << (BITS - 1)) - 1;
    __half hscale = __half();
    float inv = 0.f;
    if (MODE == 0) {
        hscale = __float2half(__ldg(p.scale));
    } else if (MODE == 1) {
        inv = __fdiv_rn(1.0f, __ldg(p.scale + row));
    } else {
        amax = block_reduce(amax, true, scratch);
        const float s = amax > 0.f ? __fdiv_rn(amax, (float)qmax) : 1.0f; // an all-zero row quantises to zeros with scale 1
        if (threadIdx.x == 0 && p.row_scale_out)
            p.row_scale_out[row] = s;
        inv = __fdiv_rn(1.0f, s);
    }
#pragma unroll
    for (int r = 0; r < kNormRuns; ++r) {
        const int run = threadIdx.x + r * kNormThreads;
        if (run < kw) {
            uint32_t rr[8] = { 0, 0, 0, 0, 0, 0, 0, 0 };
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const uint32_t w[4] = { v[r][i].x, v[r][i].y, v[r][i].z, v[r][i].w };
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    const __half h = __ushort_as_half((unsigned short)(w[e >> 1] >> ((e & 1) * 16)));
                    int q;
                    if (MODE == 0) {
                        q = __half2int_rz(__hmul(h, hscale));
                    } else {
                        q = __float2int_rn(__fmul_rn(__half2float(h), inv));
                        q = max(qmin, min(qmax, q));
                    }
                    const int pos = 31 - (8 * i + e); // byte y of rr[s] holds element 31 - 8y - s (what bytes_to_planes expects)
                    rr[pos & 7] |= ((uint32_t)q & 0xffu) << (8 * (pos >> 3));
                }
            }
            uint32_t pl[BITS];
            bytes_to_planes<BITS>(rr, pl);
#pragma unroll
            for (int b = 0; b < BITS; ++b)
                p.planes[(long)b * L + (long)row * kw + run] = pl[b];
        }
    }
}

template <int BITS>
static cudaError_t launch_prenorm(const PrenormArgs &p, int mode, cudaStream_t stream)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)p.rows);
    cfg.blockDim = dim3(kNormThreads);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    switch (mode) {
    case 0: return cudaLaunchKernelEx(&cfg, rmsnorm_quantize_pack_kernel<BITS, 0>, p);
    case 1: return cudaLaunchKernelEx(&cfg, rmsnorm_quantize_pack_kernel<BITS, 1>, p);
    default: return cudaLaunchKernelEx(&cfg, rmsnorm_quantize_pack_kernel<BITS, 2>, p);
    }
}

} // namespace abq

extern "C" abq_status abq_rmsnorm_quantize_pack_half(const void *x_half, const void *residual_half, void *sum_out_half, const void *gamma_half,
                                                     float eps, const float *scale, float *row_scale_out, void *planes, void *y_out_half, int rows,
                                                     int K, int bits, int mode, abq_stream_t stream)
{
    using namespace abq;
    if (!x_half || !gamma_half || rows <= 0 || K < 128 || K % 128 != 0 || K > 32 * kNormThreads * kNormRuns || bits < 1 || bits > 8 || mode < 0 ||
        mode > 2)
        return ABQ_ERR_INVALID_ARG;
    if (!planes && !y_out_half && !(residual_half && sum_out_half))
        return ABQ_ERR_INVALID_ARG; // nothing to write
    if (planes && ((mode == 0 || mode == 1) && !scale))
        return ABQ_ERR_INVALID_ARG;
    if (planes && mode == 2 && !row_scale_out)
        return ABQ_ERR_INVALID_ARG; // the GEMM's epilogue needs the scales this call chose
    const uintptr_t all = reinterpret_cast<uintptr_t>(x_half) | reinterpret_cast<uintptr_t>(residual_half) | reinterpret_cast<uintptr_t>(sum_out_half) |
                          reinterpret_cast<uintptr_t>(gamma_half) | reinterpret_cast<uintptr_t>(y_out_half);
    if ((all & 15) || (reinterpret_cast<uintptr_t>(planes) & 3))
        return ABQ_ERR_INVALID_ARG;
    PrenormArgs p;
    p.a = reinterpret_cast<const __half *>(x_half);
    p.b = reinterpret_cast<const __half *>(residual_half);
    p.sum_out = reinterpret_cast<__half *>(sum_out_half);
    p.gamma = reinterpret_cast<const __half *>(gamma_half);
    p.eps = eps;
    p.scale = scale;
    p.row_scale_out = row_scale_out;
    p.planes = reinterpret_cast<uint32_t *>(planes);
    p.y_out = reinterpret_cast<__half *>(y_out_half);
    p.rows = rows;
    p.K = K;
    cudaError_t e;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    switch (bits) {
    case 1: e = launch_prenorm<1>(p, mode, st); break;
    case 2: e = launch_prenorm<2>(p, mode, st); break;
    case 3: e = launch_prenorm<3>(p, mode, st); break;
    case 4: e = launch_prenorm<4>(p, mode, st); break;
    case 5: e = launch_prenorm<5>(p, mode, st); break;
    case 6: e = launch_prenorm<6>(p, mode, st); break;
    case 7: e = launch_prenorm<7>(p, mode, st); break;
    default: e = launch_prenorm<8>(p, mode, st); break;
    }
    if (e != cudaSuccess) {
        set_last_cuda_error(e);
        return ABQ_ERR_CUDA;
    }
    return ABQ_OK;
}
