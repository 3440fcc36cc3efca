// Plane -> byte expansion kernels that feed the integer tensor-core routes.
//
//  * unpack_i8:      planes[bits][rows][K/32] -> int8/uint8 codes [rows][K] (row-major, K contiguous);
//                    operand format of the tcgen05 route.
//  * xprep_decode:   activation planes -> per-128-group "records" holding the mma.sync B fragments of
//                    the decode route in exactly the order its warps read them, plus per-group code sums
//                    (needed for zero points and for two's complement weights handled as offset codes).
//
// The reference has no counterpart: it feeds the planes themselves to 1-bit tensor-core MMAs
// (engine/mma_any/aq_bmma_kernel.h:227-251), an instruction class that sm_100a only emulates.
#include "abq_common.cuh"
#include "abq_kernels.h"

namespace abq {

// 4x4 byte transpose helpers: out_y = (a.y, b.y, c.y, d.y) as bytes 0..3.
__device__ __forceinline__ void transpose4(uint32_t a, uint32_t b, uint32_t c, uint32_t d, uint32_t (&o)[4])
{
    const uint32_t u0 = __byte_perm(a, b, 0x5140), u1 = __byte_perm(a, b, 0x7362);
    const uint32_t v0 = __byte_perm(c, d, 0x5140), v1 = __byte_perm(c, d, 0x7362);
    o[0] = __byte_perm(u0, v0, 0x5410);
    o[1] = __byte_perm(u0, v0, 0x7632);
    o[2] = __byte_perm(u1, v1, 0x5410);
    o[3] = __byte_perm(u1, v1, 0x7632);
}

template <int BITS>
__global__ void __launch_bounds__(256) unpack_i8_kernel(const uint32_t *__restrict__ planes, uint32_t *__restrict__ out, long L,
                                                        int is_signed)
{
    const long idx = (long)blockIdx.x * 256 + threadIdx.x; // one 32-element run per thread
    if (idx >= L)
        return;
    uint32_t p[BITS];
#pragma unroll
    for (int b = 0; b < BITS; ++b)
        p[b] = __ldg(planes + (long)b * L + idx);
    uint32_t r[8];
    planes_to_bytes<BITS>(p, false, r);
    if (is_signed && BITS < 8) {
#pragma unroll
        for (int s = 0; s < 8; ++s)
            r[s] = sign_extend_bytes(r[s], BITS);
    }
    // byte y of r[s] is element 31 - 8y - s.  Output word (7 - 2y) holds elements 28-8y .. 31-8y =
    // (r3.y, r2.y, r1.y, r0.y); word (6 - 2y) holds (r7.y, r6.y, r5.y, r4.y).
    uint32_t hi[4], lo[4];
    transpose4(r[3], r[2], r[1], r[0], hi);
    transpose4(r[7], r[6], r[5], r[4], lo);
    uint4 *dst = reinterpret_cast<uint4 *>(out + idx * 8);
    dst[0] = make_uint4(lo[3], hi[3], lo[2], hi[2]);
    dst[1] = make_uint4(lo[1], hi[1], lo[0], hi[0]);
}

cudaError_t unpack_i8(const uint32_t *planes, void *out, int rows, int K, int bits, int is_signed, cudaStream_t stream)
{
    const long L = (long)rows * (K / 32);
    const unsigned blocks = (unsigned)((L + 255) / 256);
#define CALL(B) (unpack_i8_kernel<B><<<blocks, 256, 0, stream>>>(planes, reinterpret_cast<uint32_t *>(out), L, is_signed), cudaGetLastError())
    switch (bits) {
    case 1: return CALL(1);
    case 2: return CALL(2);
    case 3: return CALL(3);
    case 4: return CALL(4);
    case 5: return CALL(5);
    case 6: return CALL(6);
    case 7: return CALL(7);
    case 8: return CALL(8);
    default: return cudaErrorInvalidValue;
    }
#undef CALL
}

// Decode-route activation records.  For 128-group G (k in [128G, 128G+128)) the record is
//   [ token tile mt ][ step pair ip = 0..1 ][ lane = 4*g + t ][ 16 bytes ]   (B fragments, 512 B per pair)
//   [ int32 code sums of the group for tokens 0..15 ]                        (64 B)
// The 16 bytes of (mt, ip, lane) are the registers (b0, b1) of MMA step 2 ip and (b0, b1) of step 2 ip + 1 of
// mma.sync.m16n8k32 for token 8*mt + g, i.e. registers r[4 ip .. 4 ip + 3] where byte y of r[s] is
// x[token][128 G + 32 t + 31 - 8 y - s]; the weight side expands its planes into the matching k order
// (expand.cuh, gemm_decode.cu).
// One thread per (padded token, 32-element run); tokens >= M give zero fragments and zero sums.
template <int BITS>
__global__ void __launch_bounds__(128) xprep_decode_kernel(const uint32_t *__restrict__ xplanes, uint8_t *__restrict__ records,
                                                           int *__restrict__ counters, int n_counters, int M, int KW, int MT, int x_signed)
{
    // Let the GEMM that follows start early (it prefetches weights, then waits for this grid); the
    // records themselves may still be read by the previous GEMM in the stream, so wait before writing.
    pdl_launch_dependents();
    pdl_wait_prior_grid();
    const int rec_bytes = decode_record_bytes(MT);
    const long idx = (long)blockIdx.x * 128 + threadIdx.x;
    const long total = (long)MT * 8 * KW;
    for (long i = idx; i < n_counters; i += (long)gridDim.x * 128)
        counters[i] = 0; // split-K arrival counters of the GEMM that follows
    const int m = (int)(idx / KW), kw = (int)(idx % KW);
    const bool active = idx < total;
    uint32_t r[8];
#pragma unroll
    for (int s = 0; s < 8; ++s)
        r[s] = 0;
    int sum = 0;
    if (active && m < M) {
        uint32_t p[BITS];
        const long L = (long)M * KW;
#pragma unroll
        for (int b = 0; b < BITS; ++b)
            p[b] = __ldg(xplanes + (long)b * L + (long)m * KW + kw);
        planes_to_bytes<BITS>(p, false, r);
        if (x_signed && BITS < 8) {
#pragma unroll
            for (int s = 0; s < 8; ++s)
                r[s] = sign_extend_bytes(r[s], BITS);
        }
        if (x_signed) {
#pragma unroll
            for (int s = 0; s < 8; ++s)
                sum = __dp4a((int)r[s], 0x01010101, sum);
        } else {
            unsigned usum = 0;
#pragma unroll
            for (int s = 0; s < 8; ++s)
                usum = __dp4a(r[s], 0x01010101u, usum);
            sum = (int)usum;
        }
    }
    // the four runs of a 128-group sit in four consecutive lanes
    sum += __shfl_xor_sync(0xffffffffu, sum, 1);
    sum += __shfl_xor_sync(0xffffffffu, sum, 2);
    if (!active)
        return;
    const int G = kw >> 2, t = kw & 3, mt = m >> 3, g = m & 7;
    uint8_t *rec = records + (long)G * rec_bytes;
#pragma unroll
    for (int ip = 0; ip < 2; ++ip) {
        uint4 *dst = reinterpret_cast<uint4 *>(rec + ((mt * 2 + ip) * 32 + g * 4 + t) * 16);
        *dst = make_uint4(r[4 * ip], r[4 * ip + 1], r[4 * ip + 2], r[4 * ip + 3]);
    }
    if (t == 0)
        reinterpret_cast<int *>(rec + 1024 * MT)[m] = sum;
    if (MT == 1 && t == 1) // tokens 8..15 of the sum block are unused with one token tile: keep them defined
        reinterpret_cast<int *>(rec + 1024 * MT)[8 + m] = 0;
}

cudaError_t xprep_decode(const uint32_t *xplanes, void *records, int *counters, int n_counters, int M, int K, int bits, int x_signed,
                         int MT, bool pdl, cudaStream_t stream)
{
    const int KW = K / 32;
    const long total = (long)MT * 8 * KW;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)((total + 127) / 128));
    cfg.blockDim = dim3(128);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    uint8_t *rec = reinterpret_cast<uint8_t *>(records);
#define CALL(B) cudaLaunchKernelEx(&cfg, xprep_decode_kernel<B>, xplanes, rec, counters, n_counters, M, KW, MT, x_signed)
    switch (bits) {
    case 1: return CALL(1);
    case 2: return CALL(2);
    case 3: return CALL(3);
    case 4: return CALL(4);
    case 5: return CALL(5);
    case 6: return CALL(6);
    case 7: return CALL(7);
    case 8: return CALL(8);
    default: return cudaErrorInvalidValue;
    }
#undef CALL
}

} // namespace abq
