// Quantise-on-load: fp16 weights [N][K] -> unsigned codes as bit-planes (the layout abq_pack_int32 writes and the GEMM
// routes read) + fp16 scale + u8 zero point per output channel or per group of input features.
//
// Restates the min/max calibration of the reference's UniformAffineQuantizer (algorithm/quantize/quantizer.py:149-179,
// without learnable clipping) and its code rule (quantizer.py:111-132) in fp32:
//     asymmetric: scale = clamp((max - min) / L, 1e-5, 1e4),  L = 2^bits - 1 (2^bits for 1 and 2 bits, quantizer.py:170-171)
//                 zero  = rint(clamp(-min / scale, -1e4, 1e4))
//     symmetric:  scale = clamp(absmax / (2^(bits-1) - 1), 1e-5, 1e4),  zero = 2^(bits-1) - 1   (quantizer.py:163-167)
//     code = clamp(rint(x / scale) + zero, 0, 2^bits - 1)
// Two deliberate differences, both because `bits` planes hold the codes 0 .. 2^bits - 1 and nothing else: the reference
// lets 1- and 2-bit codes reach 2^bits (its "bit balance", quantizer.py:66-68) and lets the zero point leave the code
// range; here both are clamped into it.  Groups are contiguous runs of `group_size` input features (quantizer.py:116-119).
//
// One CTA per weight row.  A thread owns 32-feature runs (64 bytes, four 16-byte loads); run minima / maxima meet in
// shared memory, every thread then reads the range of its group (or of the row), quantises its runs and writes one word
// per plane -- each fp16 value is read twice (the second time from L2), each plane word written once.
#include <cuda_fp16.h>

#include "abq_common.cuh"
#include "abq_kernels.h"

namespace abq {

constexpr int kWquantThreads = 128;

__device__ __forceinline__ void load_run(const __half *row, int run, float (&v)[32])
{
    const uint4 *src = reinterpret_cast<const uint4 *>(row + (size_t)run * 32);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint4 q = __ldg(src + i);
        const uint32_t w[4] = { q.x, q.y, q.z, q.w };
#pragma unroll
        for (int e = 0; e < 8; ++e)
            v[8 * i + e] = __half2float(__ushort_as_half((unsigned short)(w[e >> 1] >> ((e & 1) * 16))));
    }
}

template <int BITS>
__global__ void __launch_bounds__(kWquantThreads) quantize_weights_kernel(const __half *__restrict__ w, uint32_t *__restrict__ planes,
                                                                          __half *__restrict__ scale_out, uint8_t *__restrict__ zero_out, int N, int K,
                                                                          int runs_per_group, int symmetric)
{
    extern __shared__ float run_range[]; // [2][K / 32]: minimum, maximum of every run of this row
    const int KW = K >> 5;
    const int row = blockIdx.x;
    const __half *src = w + (size_t)row * K;
    float *rmin = run_range, *rmax = run_range + KW;
    for (int run = threadIdx.x; run < KW; run += kWquantThreads) {
        float v[32];
        load_run(src, run, v);
        float lo = v[0], hi = v[0];
#pragma unroll
        for (int j = 1; j < 32; ++j) {
            lo = fminf(lo, v[j]);
            hi = fmaxf(hi, v[j]);
        }
        rmin[run] = lo;
        rmax[run] = hi;
    }
    __syncthreads();
    const int groups = KW / runs_per_group;
    const int qmax = (1 << BITS) - 1;
    const float levels = BITS <= 2 ? (float)(1 << BITS) : (float)qmax;
    for (int run = threadIdx.x; run < KW; run += kWquantThreads) {
        const int grp = run / runs_per_group;
        float lo = rmin[grp * runs_per_group], hi = rmax[grp * runs_per_group];
        for (int j = 1; j < runs_per_group; ++j) {
            lo = fminf(lo, rmin[grp * runs_per_group + j]);
            hi = fmaxf(hi, rmax[grp * runs_per_group + j]);
        }
        float scale, zero;
        if (symmetric) {
            scale = __fdiv_rn(fmaxf(fabsf(lo), fabsf(hi)), (float)((1 << (BITS - 1)) - 1));
            scale = fminf(fmaxf(scale, 1e-5f), 1e4f);
            zero = (float)((1 << (BITS - 1)) - 1);
        } else {
            scale = __fdiv_rn(__fsub_rn(hi, lo), levels);
            scale = fminf(fmaxf(scale, 1e-5f), 1e4f);
            zero = rintf(fminf(fmaxf(__fdiv_rn(-lo, scale), -1e4f), 1e4f));
            zero = fminf(fmaxf(zero, 0.f), (float)qmax);
        }
        float v[32];
        load_run(src, run, v);
        uint32_t r[8] = { 0, 0, 0, 0, 0, 0, 0, 0 };
#pragma unroll
        for (int j = 0; j < 32; ++j) {
            float c = __fadd_rn(rintf(__fdiv_rn(v[j], scale)), zero);
            c = fminf(fmaxf(c, 0.f), (float)qmax);
            const int pos = 31 - j; // byte y of r[s] holds element 31 - 8y - s of the run
            r[pos & 7] |= (uint32_t)(int)c << (8 * (pos >> 3));
        }
        uint32_t p[BITS];
        bytes_to_planes<BITS>(r, p);
#pragma unroll
        for (int b = 0; b < BITS; ++b)
            planes[((size_t)b * N + row) * KW + run] = p[b];
        if (run % runs_per_group == 0) {
            scale_out[(size_t)row * groups + grp] = __float2half_rn(scale);
            zero_out[(size_t)row * groups + grp] = (uint8_t)(int)zero;
        }
    }
}

template <int BITS>
static cudaError_t launch_wquant(const __half *w, uint32_t *planes, __half *scale, uint8_t *zero, int N, int K, int rpg, int symmetric,
                                 cudaStream_t stream)
{
    quantize_weights_kernel<BITS><<<N, kWquantThreads, (size_t)(K / 32) * 8, stream>>>(w, planes, scale, zero, N, K, rpg, symmetric);
    return cudaGetLastError();
}

cudaError_t quantize_weights(const __half *w, uint32_t *planes, __half *scale, uint8_t *zero, int N, int K, int bits, int group_size, int symmetric,
                             cudaStream_t stream)
{
    const int rpg = (group_size > 0 ? group_size : K) / 32;
    switch (bits) {
    case 1: return launch_wquant<1>(w, planes, scale, zero, N, K, rpg, symmetric, stream);
    case 2: return launch_wquant<2>(w, planes, scale, zero, N, K, rpg, symmetric, stream);
    case 3: return launch_wquant<3>(w, planes, scale, zero, N, K, rpg, symmetric, stream);
    case 4: return launch_wquant<4>(w, planes, scale, zero, N, K, rpg, symmetric, stream);
    case 5: return launch_wquant<5>(w, planes, scale, zero, N, K, rpg, symmetric, stream);
    case 6: return launch_wquant<6>(w, planes, scale, zero, N, K, rpg, symmetric, stream);
    case 7: return launch_wquant<7>(w, planes, scale, zero, N, K, rpg, symmetric, stream);
    case 8: return launch_wquant<8>(w, planes, scale, zero, N, K, rpg, symmetric, stream);
    }
    return cudaErrorInvalidValue;
}

} // namespace abq
