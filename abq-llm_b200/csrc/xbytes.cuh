// Activation side shared by the decode kernels: bit-planes (or fp16 values) of 32 consecutive activation codes -> the
// eight registers of byte codes that the int8 MMA B fragments are cut from.
#pragma once
#include <cuda_fp16.h>
#include <stdint.h>

#include "abq_common.cuh"
#include "expand.cuh"

namespace abq {

// Bit-planes of 32 activation codes -> eight registers of true byte values (byte y of r[s] = code at bit 8y + s).
template <int P>
__device__ __forceinline__ void x_bytes(const uint32_t (&p)[P], bool is_signed, uint32_t (&r)[8])
{
    if constexpr (P >= 5 || P == 1) {
        Expand<P>::run(p, r); // these widths come out of the butterfly as plain byte values
    } else {
        uint32_t n[4];
        if constexpr (P == 2)
            nibble_fields(p[0], p[1], 0u, 0u, false, n);
        else if constexpr (P == 3)
            nibble_fields(p[0], p[1], p[2], 0u, false, n);
        else
            nibble_fields(p[0], p[1], p[2], p[3], true, n);
#pragma unroll
        for (int s = 0; s < 4; ++s) {
            r[s] = n[s] & 0x0f0f0f0fu;
            r[4 + s] = (n[s] >> 4) & 0x0f0f0f0fu;
        }
    }
    if (is_signed && P < 8) {
#pragma unroll
        for (int s = 0; s < 8; ++s)
            r[s] = sign_extend_bytes(r[s], P);
    }
}

// The same eight registers straight from 32 fp16 activations: code = (int)(half(x) * half(scale)), truncated, the low
// `bits` bits kept and sign-extended -- the FasterTransformer wrapper's quantiser (abq_gemm_wrapper.cu:29-54) without
// the round trip through planes.  `src` points to the 32 halves (64 bytes, 16-byte aligned).
__device__ __forceinline__ void x_bytes_from_half(const uint4 *src, __half hscale, int bits, uint32_t (&r)[8])
{
#pragma unroll
    for (int s = 0; s < 8; ++s)
        r[s] = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint4 v = __ldg(src + i);
        const uint32_t w[4] = { v.x, v.y, v.z, v.w };
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const __half h = __ushort_as_half((unsigned short)(w[e >> 1] >> ((e & 1) * 16)));
            const uint32_t code = (uint32_t)__half2int_rz(__hmul(h, hscale)) & 0xffu;
            const int pos = 31 - (8 * i + e); // byte y of r[s] holds element 31 - 8y - s of the run
            r[pos & 7] |= code << (8 * (pos >> 3));
        }
    }
    const uint32_t keep = 0x01010101u * ((1u << bits) - 1u);
#pragma unroll
    for (int s = 0; s < 8; ++s) {
        r[s] &= keep;
        if (bits < 8)
            r[s] = sign_extend_bytes(r[s], bits);
    }
}

} // namespace abq
