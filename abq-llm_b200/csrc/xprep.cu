// Plane -> byte expansion kernels that feed the integer tensor-core routes.
//
//  * unpack_i8:      planes[bits][rows][K/32] -> int8/uint8 codes [rows][K] (row-major, K contiguous);
//                    operand format of the tcgen05 route.  (The decode route expands its activation planes
//                    inside the GEMM kernel, see gemm_decode.cu.)
//
// The reference has no counterpart: it feeds the planes themselves to 1-bit tensor-core MMAs
// (engine/mma_any/aq_bmma_kernel.h:227-251), an instruction class that sm_100a only emulates.
#include <cuda_fp16.h>

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

// 32-element runs, one per lane and step: BITS plane words -> 32 code bytes in element order.  Called by whole warps
// (runs past the end are skipped lane by lane): neighbouring lanes swap halves so that every store instruction writes complete 32-byte
// sectors (each lane alone would write its 32 bytes as two half sectors).
constexpr int kUnpackRuns = 4; // runs per thread, 256 threads apart: all their plane loads are in flight before the first is used

// Optional zero points: `zero` [rows][zgroups] bytes, one per run of `zwords` plane words of a row of `kw` words; the
// codes written are then code - zero (two's complement bytes; the caller guarantees that the difference fits int8).
struct ZeroTable {
    const uint8_t *zero;
    int kw, zwords, zgroups;
};

template <int BITS>
__device__ __forceinline__ void unpack_run(const uint32_t *__restrict__ planes, uint32_t *__restrict__ out, long L, long idx0, int is_signed,
                                           const ZeroTable zt = ZeroTable{ nullptr, 0, 0, 0 })
{
    uint32_t p[kUnpackRuns][BITS];
    bool live[kUnpackRuns];
#pragma unroll
    for (int u = 0; u < kUnpackRuns; ++u) {
        const long idx = idx0 + u * 256;
        live[u] = idx < L;
#pragma unroll
        for (int b = 0; b < BITS; ++b)
            p[u][b] = live[u] ? __ldg(planes + (long)b * L + idx) : 0u;
    }
#pragma unroll
    for (int u = 0; u < kUnpackRuns; ++u) {
        const long idx = idx0 + u * 256;
        uint32_t r[8];
        planes_to_bytes<BITS>(p[u], false, r);
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
        uint4 q0 = make_uint4(lo[3], hi[3], lo[2], hi[2]), q1 = make_uint4(lo[1], hi[1], lo[0], hi[0]);
        if (zt.zero && live[u]) { // the 32 codes of a run share their scale group
            const long row = idx / zt.kw;
            const uint32_t zz = 0x01010101u * zt.zero[row * zt.zgroups + (int)(idx - row * zt.kw) / zt.zwords];
            q0 = make_uint4(__vsub4(q0.x, zz), __vsub4(q0.y, zz), __vsub4(q0.z, zz), __vsub4(q0.w, zz));
            q1 = make_uint4(__vsub4(q1.x, zz), __vsub4(q1.y, zz), __vsub4(q1.z, zz), __vsub4(q1.w, zz));
        }
        const bool odd = threadIdx.x & 1;
        const uint4 give = odd ? q0 : q1; // the even lane hands over its second half, the odd lane its first half
        uint4 got;
        got.x = __shfl_xor_sync(0xffffffffu, give.x, 1);
        got.y = __shfl_xor_sync(0xffffffffu, give.y, 1);
        got.z = __shfl_xor_sync(0xffffffffu, give.z, 1);
        got.w = __shfl_xor_sync(0xffffffffu, give.w, 1);
        if (live[u]) { // L is even and lane pairs are aligned: a live lane's neighbour is live
            uint4 *pair = reinterpret_cast<uint4 *>(out + (idx & ~1L) * 8); // 64 bytes of the lane pair: [even q0][even q1][odd q0][odd q1]
            pair[odd ? 1 : 0] = odd ? got : q0;
            pair[odd ? 3 : 2] = odd ? q1 : got;
        }
    }
}

__device__ __forceinline__ void unpack_any(const uint32_t *planes, uint32_t *out, long L, long idx, int bits, int is_signed,
                                           const ZeroTable zt = ZeroTable{ nullptr, 0, 0, 0 })
{
    switch (bits) { // uniform per block
    case 1: unpack_run<1>(planes, out, L, idx, is_signed, zt); break;
    case 2: unpack_run<2>(planes, out, L, idx, is_signed, zt); break;
    case 3: unpack_run<3>(planes, out, L, idx, is_signed, zt); break;
    case 4: unpack_run<4>(planes, out, L, idx, is_signed, zt); break;
    case 5: unpack_run<5>(planes, out, L, idx, is_signed, zt); break;
    case 6: unpack_run<6>(planes, out, L, idx, is_signed, zt); break;
    case 7: unpack_run<7>(planes, out, L, idx, is_signed, zt); break;
    default: unpack_run<8>(planes, out, L, idx, is_signed, zt); break;
    }
}

template <int BITS>
__global__ void __launch_bounds__(256) unpack_i8_kernel(const uint32_t *__restrict__ planes, uint32_t *__restrict__ out, long L,
                                                        int is_signed, const ZeroTable zt)
{
    pdl_launch_dependents(); // a GEMM kernel launched programmatically behind this one may start its set-up
    unpack_run<BITS>(planes, out, L, (long)blockIdx.x * (256 * kUnpackRuns) + threadIdx.x, is_signed, zt);
}

// Both operands of a GEMM in one launch: blocks [0, blocks_a) expand operand a, the rest operand b.  Lets the
// dependent GEMM kernel start its set-up early (programmatic launch) and saves a launch per GEMM.
__global__ void __launch_bounds__(256) unpack_pair_kernel(const uint32_t *__restrict__ pa, uint32_t *__restrict__ oa, long La, int bits_a,
                                                          int signed_a, unsigned blocks_a, const uint32_t *__restrict__ pb,
                                                          uint32_t *__restrict__ ob, long Lb, int bits_b, int signed_b, const ZeroTable zt_b)
{
    pdl_launch_dependents();
    if (blockIdx.x < blocks_a) {
        unpack_any(pa, oa, La, (long)blockIdx.x * (256 * kUnpackRuns) + threadIdx.x, bits_a, signed_a);
    } else {
        unpack_any(pb, ob, Lb, (long)(blockIdx.x - blocks_a) * (256 * kUnpackRuns) + threadIdx.x, bits_b, signed_b, zt_b);
    }
}

cudaError_t unpack_pair_i8(const uint32_t *planes_a, void *out_a, int rows_a, int bits_a, int signed_a, const uint32_t *planes_b, void *out_b,
                           int rows_b, int bits_b, int signed_b, int K, cudaStream_t stream, const uint8_t *zero_b, int zero_group)
{
    const ZeroTable zt = { zero_b, K / 32, zero_b ? zero_group / 32 : 1, zero_b ? K / zero_group : 1 };
    const long La = (long)rows_a * (K / 32), Lb = (long)rows_b * (K / 32);
    const long per = 256 * kUnpackRuns;
    const unsigned blocks_a = (unsigned)((La + per - 1) / per), blocks_b = (unsigned)((Lb + per - 1) / per);
    unpack_pair_kernel<<<blocks_a + blocks_b, 256, 0, stream>>>(planes_a, reinterpret_cast<uint32_t *>(out_a), La, bits_a, signed_a, blocks_a,
                                                                planes_b, reinterpret_cast<uint32_t *>(out_b), Lb, bits_b, signed_b, zt);
    return cudaGetLastError();
}

// fp16 activations -> int8 codes [rows][K], the static-scale quantiser of the FasterTransformer wrapper
// (abq_gemm_wrapper.cu:29-54): code = (int)(half(x) * half(scale[0])), truncated, the low `bits` bits kept and
// sign-extended.  16 values per thread: two 16-byte loads, one 16-byte store.
__global__ void __launch_bounds__(256) quantize_codes_kernel(const __half *__restrict__ in, const float *__restrict__ scale,
                                                             uint4 *__restrict__ out, long n16, int bits)
{
    pdl_launch_dependents();
    const long idx = (long)blockIdx.x * 256 + threadIdx.x;
    if (idx >= n16)
        return;
    const __half hscale = __float2half(__ldg(scale));
    const uint32_t keep = 0x01010101u * ((1u << bits) - 1u);
    const uint4 *src = reinterpret_cast<const uint4 *>(in) + idx * 2;
    uint32_t o[4] = { 0, 0, 0, 0 };
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const uint4 v = __ldg(src + i);
        const uint32_t w[4] = { v.x, v.y, v.z, v.w };
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const __half h = __ushort_as_half((unsigned short)(w[e >> 1] >> ((e & 1) * 16)));
            const uint32_t code = (uint32_t)__half2int_rz(__hmul(h, hscale)) & 0xffu;
            o[2 * i + (e >> 2)] |= code << (8 * (e & 3));
        }
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        o[k] &= keep;
        if (bits < 8)
            o[k] = sign_extend_bytes(o[k], bits);
    }
    out[idx] = make_uint4(o[0], o[1], o[2], o[3]);
}

cudaError_t quantize_codes(const void *in_half, const float *scale, void *out, int rows, int K, int bits, cudaStream_t stream)
{
    const long n16 = (long)rows * K / 16;
    quantize_codes_kernel<<<(unsigned)((n16 + 255) / 256), 256, 0, stream>>>(reinterpret_cast<const __half *>(in_half), scale,
                                                                             reinterpret_cast<uint4 *>(out), n16, bits);
    return cudaGetLastError();
}

cudaError_t unpack_i8(const uint32_t *planes, void *out, int rows, int K, int bits, int is_signed, cudaStream_t stream, const uint8_t *zero,
                      int zero_group)
{
    const ZeroTable zt = { zero, K / 32, zero ? zero_group / 32 : 1, zero ? K / zero_group : 1 };
    const long L = (long)rows * (K / 32);
    const unsigned blocks = (unsigned)((L + 256 * kUnpackRuns - 1) / (256 * kUnpackRuns));
#define CALL(B) (unpack_i8_kernel<B><<<blocks, 256, 0, stream>>>(planes, reinterpret_cast<uint32_t *>(out), L, is_signed, zt), cudaGetLastError())
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
