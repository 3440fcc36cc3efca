// Bit-plane packing kernels: value tensors -> planes[bit][rows][K/32], element j of a 32-run at bit 31-j.
//
// Replaces the reference's `pack` / `pack4` (engine/common/pack.cu:18-64) and the FasterTransformer
// wrapper's `pack_half` (fastertransformer/.../abqgemm/abq_gemm_wrapper.cu:29-54).  The reference
// launches one block row per plane, so the input is re-read (and for fp16 re-quantised) once per
// plane; here every value is read once: a thread loads one run of 32 consecutive values with
// 16-byte loads, quantises them, collects the code bytes in eight registers and transposes them into
// the plane words in registers (two operations per byte register and plane); consecutive threads
// write consecutive words of every plane.  (A ballot per plane and run, the first version, was bound
// by the vote instruction: 15 % of the HBM rate for 8-bit activations.)
#include "abq_common.cuh"

namespace abq {

constexpr int kPackThreads = 256;

// Place the low byte of code j (element index in the run) where bytes_to_planes expects it: byte y of r[s] holds
// element 31 - 8y - s.
__device__ __forceinline__ void put_code(uint32_t (&r)[8], int j, uint32_t code)
{
    const int pos = 31 - j, s = pos & 7, y = pos >> 3;
    r[s] |= (code & 0xffu) << (8 * y);
}

// One thread per output word (= 32 codes = 128 bytes of input).  `L` = rows * K / 32 words per plane.
// A thread that fetched its own 128 bytes would make every load instruction of the warp touch 32 different lines (256
// L1 wavefronts per 4 KB: the kernel then stops at about 4.5 TB/s of input whatever the DRAM does), so a warp fetches
// its 4 KB with consecutive lanes on consecutive 16-byte chunks and hands them over through shared memory, chunk
// position XOR run index so that both the stores and the per-run reads are free of bank conflicts.
template <int BITS>
__global__ void __launch_bounds__(kPackThreads) pack_int32_kernel(const int32_t *__restrict__ in, uint32_t *__restrict__ planes,
                                                                  long L)
{
    __shared__ int4 stage[kPackThreads * 8];
    const int lane = threadIdx.x & 31;
    const long idx = (long)blockIdx.x * kPackThreads + threadIdx.x;
    const long warp_run0 = idx - lane;
    int4 *mine = stage + (threadIdx.x - lane) * 8; // this warp's 256 chunks
    const int4 *src = reinterpret_cast<const int4 *>(in) + warp_run0 * 8;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int c = i * 32 + lane, run = c >> 3, pos = c & 7;
        if (warp_run0 + run < L)
            mine[run * 8 + (pos ^ (run & 7))] = __ldg(src + c);
    }
    __syncwarp();
    if (idx >= L)
        return;
    int4 v[8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
        v[i] = mine[lane * 8 + (i ^ (lane & 7))];
    uint32_t r[8] = { 0, 0, 0, 0, 0, 0, 0, 0 };
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        put_code(r, 4 * i + 0, (uint32_t)v[i].x);
        put_code(r, 4 * i + 1, (uint32_t)v[i].y);
        put_code(r, 4 * i + 2, (uint32_t)v[i].z);
        put_code(r, 4 * i + 3, (uint32_t)v[i].w);
    }
    uint32_t p[BITS];
    bytes_to_planes<BITS>(r, p);
#pragma unroll
    for (int b = 0; b < BITS; ++b)
        planes[(long)b * L + idx] = p[b];
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

// fp16 -> code -> planes, one thread per run of 32 halves (four 16-byte loads).
// MODE 0: code = (int)(h * half(scale[0])) (fp16 multiply, truncation, no clamp);
// MODE 1: code = clamp(rint(float(h) * (1 / scale[row])), -2^(bits-1), 2^(bits-1) - 1).
template <int BITS, int MODE>
__global__ void __launch_bounds__(kPackThreads) quantize_pack_half_kernel(const __half *__restrict__ in,
                                                                          const float *__restrict__ scale,
                                                                          uint32_t *__restrict__ planes, long L, int kw_per_row)
{
    const long idx = (long)blockIdx.x * kPackThreads + threadIdx.x;
    if (idx >= L)
        return;
    const uint4 *src = reinterpret_cast<const uint4 *>(in + idx * 32);
    uint4 v[4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
        v[i] = __ldg(src + i);
    const __half hscale = (MODE == 0) ? __float2half(__ldg(scale)) : __half();
    const float inv = (MODE == 1) ? __fdiv_rn(1.0f, __ldg(scale + idx / kw_per_row)) : 0.f;
    const int qmin = -(1 << (BITS - 1)), qmax = (1 << (BITS - 1)) - 1;
    uint32_t r[8] = { 0, 0, 0, 0, 0, 0, 0, 0 };
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t w[4] = { v[i].x, v[i].y, v[i].z, v[i].w };
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
            put_code(r, 8 * i + e, (uint32_t)q);
        }
    }
    uint32_t p[BITS];
    bytes_to_planes<BITS>(r, p);
#pragma unroll
    for (int b = 0; b < BITS; ++b)
        planes[(long)b * L + idx] = p[b];
}

template <int BITS>
static cudaError_t launch_pack_int32(const int32_t *in, uint32_t *planes, long L, cudaStream_t stream)
{
    const unsigned blocks = (unsigned)((L + kPackThreads - 1) / kPackThreads);
    pack_int32_kernel<BITS><<<blocks, kPackThreads, 0, stream>>>(in, planes, L);
    return cudaGetLastError();
}

template <int BITS>
static cudaError_t launch_quant_half(const __half *in, const float *scale, uint32_t *planes, long L, int kw, int mode,
                                     cudaStream_t stream)
{
    const unsigned blocks = (unsigned)((L + kPackThreads - 1) / kPackThreads);
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
