// Bit-plane packing kernels: value tensors -> planes[bit][rows][K/32], element j of a 32-run at bit 31-j.
//
// Replaces the reference's `pack` / `pack4` (engine/common/pack.cu:18-64) and the FasterTransformer
// wrapper's `pack_half` (fastertransformer/.../abqgemm/abq_gemm_wrapper.cu:29-54).  The reference
// launches one block row per plane, so the input is re-read (and for fp16 re-quantised) once per
// plane; here every value is read once: a warp loads 32 consecutive codes with one coalesced
// request, one __ballot_sync per plane turns them into a plane word, and the words of 32 consecutive
// runs are collected across lanes so that every plane is written with full 128-byte stores.
#include "abq_common.cuh"

namespace abq {

constexpr int kPackThreads = 256;

// One warp per 32 consecutive output words (= 1024 codes).  `L` = rows * K / 32 words per plane.
template <int BITS>
__global__ void __launch_bounds__(kPackThreads) pack_int32_kernel(const int32_t *__restrict__ in, uint32_t *__restrict__ planes,
                                                                  long L)
{
    const int lane = threadIdx.x & 31;
    const long warp = (long)blockIdx.x * (kPackThreads / 32) + (threadIdx.x >> 5);
    const long w0 = warp * 32;
    if (w0 >= L)
        return;
    const int nwords = (int)min((long)32, L - w0);
    uint32_t keep[BITS];
#pragma unroll
    for (int b = 0; b < BITS; ++b)
        keep[b] = 0;
    const int32_t *src = in + w0 * 32;
    for (int c = 0; c < nwords; c += 4) {
        int32_t v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u)
            v[u] = (c + u < nwords) ? __ldg(src + (long)(c + u) * 32 + lane) : 0;
#pragma unroll
        for (int u = 0; u < 4; ++u) {
#pragma unroll
            for (int b = 0; b < BITS; ++b) {
                uint32_t word = __brev(__ballot_sync(0xffffffffu, (v[u] >> b) & 1));
                if (lane == c + u)
                    keep[b] = word;
            }
        }
    }
    if (lane < nwords) {
#pragma unroll
        for (int b = 0; b < BITS; ++b)
            planes[(long)b * L + w0 + lane] = keep[b];
    }
}

// Nibble-packed 4-bit codes: one thread per output word, 16-byte load (first element = top nibble).
__global__ void __launch_bounds__(kPackThreads) pack_int4_kernel(const uint4 *__restrict__ in, uint32_t *__restrict__ planes, long L,
                                                                 int bits)
{
    const long idx = (long)blockIdx.x * kPackThreads + threadIdx.x;
    if (idx >= L)
        return;
    const uint4 v = __ldg(in + idx);
    const uint32_t w32[4] = { v.x, v.y, v.z, v.w };
    for (int b = 0; b < bits; ++b) {
        uint32_t word = 0;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            // nibble n (bits 4n..4n+3) of w32[c] is element 8c + 7 - n -> output bit 24 - 8c + n
            uint32_t x = (w32[c] >> b) & 0x11111111u;
            uint32_t byte = 0;
#pragma unroll
            for (int n = 0; n < 8; ++n)
                byte |= ((x >> (4 * n)) & 1u) << n;
            word |= byte << (24 - 8 * c);
        }
        planes[(long)b * L + idx] = word;
    }
}

// fp16 -> code -> planes.  A warp covers 64 consecutive halves per step with one half2 load per lane;
// two shuffles hand lane l the elements l and 32+l, so that one ballot yields one finished plane word.
// MODE 0: code = (int)(h * half(scale[0])) (fp16 multiply, truncation, no clamp);
// MODE 1: code = clamp(rint(float(h) * (1 / scale[row])), -2^(bits-1), 2^(bits-1) - 1).
template <int BITS, int MODE>
__global__ void __launch_bounds__(kPackThreads) quantize_pack_half_kernel(const __half *__restrict__ in,
                                                                          const float *__restrict__ scale,
                                                                          uint32_t *__restrict__ planes, long L, int kw_per_row)
{
    const int lane = threadIdx.x & 31;
    const long warp = (long)blockIdx.x * (kPackThreads / 32) + (threadIdx.x >> 5);
    const long w0 = warp * 32;
    if (w0 >= L)
        return;
    const int nwords = (int)min((long)32, L - w0); // always even: K/32 is a multiple of 4
    uint32_t keep[BITS];
#pragma unroll
    for (int b = 0; b < BITS; ++b)
        keep[b] = 0;
    const __half hscale = (MODE == 0) ? __float2half(__ldg(scale)) : __half();
    const int qmin = -(1 << (BITS - 1)), qmax = (1 << (BITS - 1)) - 1;
    const __half2 *src = reinterpret_cast<const __half2 *>(in + w0 * 32);
    for (int c = 0; c < nwords; c += 2) {
        const uint32_t raw = __ldg(reinterpret_cast<const unsigned int *>(src) + (long)c * 16 + lane);
        const uint32_t ra = __shfl_sync(0xffffffffu, raw, lane >> 1);
        const uint32_t rb = __shfl_sync(0xffffffffu, raw, 16 + (lane >> 1));
        const uint16_t ha = (lane & 1) ? (uint16_t)(ra >> 16) : (uint16_t)(ra & 0xffffu);
        const uint16_t hb = (lane & 1) ? (uint16_t)(rb >> 16) : (uint16_t)(rb & 0xffffu);
        int code[2];
        const uint16_t hv[2] = { ha, hb };
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const __half h = __ushort_as_half(hv[u]);
            if (MODE == 0) {
                code[u] = __half2int_rz(__hmul(h, hscale));
            } else {
                const long row = (w0 + c + u) / kw_per_row;
                const float inv = __fdiv_rn(1.0f, __ldg(scale + row));
                int q = __float2int_rn(__fmul_rn(__half2float(h), inv));
                code[u] = max(qmin, min(qmax, q));
            }
        }
#pragma unroll
        for (int u = 0; u < 2; ++u) {
#pragma unroll
            for (int b = 0; b < BITS; ++b) {
                uint32_t word = __brev(__ballot_sync(0xffffffffu, (code[u] >> b) & 1));
                if (lane == c + u)
                    keep[b] = word;
            }
        }
    }
    if (lane < nwords) {
#pragma unroll
        for (int b = 0; b < BITS; ++b)
            planes[(long)b * L + w0 + lane] = keep[b];
    }
}

template <int BITS>
static cudaError_t launch_pack_int32(const int32_t *in, uint32_t *planes, long L, cudaStream_t stream)
{
    const long warps = (L + 31) / 32;
    const unsigned blocks = (unsigned)((warps + kPackThreads / 32 - 1) / (kPackThreads / 32));
    pack_int32_kernel<BITS><<<blocks, kPackThreads, 0, stream>>>(in, planes, L);
    return cudaGetLastError();
}

template <int BITS>
static cudaError_t launch_quant_half(const __half *in, const float *scale, uint32_t *planes, long L, int kw, int mode,
                                     cudaStream_t stream)
{
    const long warps = (L + 31) / 32;
    const unsigned blocks = (unsigned)((warps + kPackThreads / 32 - 1) / (kPackThreads / 32));
    if (mode == 0)
        quantize_pack_half_kernel<BITS, 0><<<blocks, kPackThreads, 0, stream>>>(in, scale, planes, L, kw);
    else
        quantize_pack_half_kernel<BITS, 1><<<blocks, kPackThreads, 0, stream>>>(in, scale, planes, L, kw);
    return cudaGetLastError();
}

#define ABQ_DISPATCH_BITS(bits, CALL)                                                                                  \
    switch (bits) {                                                                                                    \
    case 1: return CALL(1);                                                                                            \
    case 2: return CALL(2);                                                                                            \
    case 3: return CALL(3);                                                                                            \
    case 4: return CALL(4);                                                                                            \
    case 5: return CALL(5);                                                                                            \
    case 6: return CALL(6);                                                                                            \
    case 7: return CALL(7);                                                                                            \
    case 8: return CALL(8);                                                                                            \
    default: return cudaErrorInvalidValue;                                                                             \
    }

cudaError_t pack_int32(const int32_t *in, uint32_t *planes, int rows, int K, int bits, cudaStream_t stream)
{
    const long L = (long)rows * (K / 32);
#define CALL(B) launch_pack_int32<B>(in, planes, L, stream)
    ABQ_DISPATCH_BITS(bits, CALL)
#undef CALL
}

cudaError_t pack_int4(const void *in, uint32_t *planes, int rows, int K, int bits, cudaStream_t stream)
{
    const long L = (long)rows * K / 32;
    const unsigned blocks = (unsigned)((L + kPackThreads - 1) / kPackThreads);
    pack_int4_kernel<<<blocks, kPackThreads, 0, stream>>>(reinterpret_cast<const uint4 *>(in), planes, L, bits);
    return cudaGetLastError();
}

cudaError_t quantize_pack_half(const __half *in, const float *scale, uint32_t *planes, int rows, int K, int bits, int mode,
                               cudaStream_t stream)
{
    const long L = (long)rows * (K / 32);
    const int kw = K / 32;
#define CALL(B) launch_quant_half<B>(in, scale, planes, L, kw, mode, stream)
    ABQ_DISPATCH_BITS(bits, CALL)
#undef CALL
}

} // namespace abq
