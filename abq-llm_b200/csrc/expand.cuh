// Bit-plane -> byte-code expansion for the decode route.
//
// Input: the Q plane words of 32 consecutive codes of one weight row (plane b in p[b]; the element stored at bit
// position u of the words is code index 31 - u).  Output: eight registers r[0..7]; byte y of r[s] is the unsigned
// code of the element at bit position 8y + s, multiplied by 2^shift(s) where shift depends only on the MMA step
// s / 2.  Steps with different shifts accumulate into different accumulator sets (kSets <= 2); the set with the
// larger scale is divided by 2^kShift when the sets are merged, which is exact.
//
// The expansion is a butterfly over bit fields (a bit-matrix transposition of the Q x 32 plane block):
//   Q = 2     : 2-bit fields, masks 0x03 / 0x0C pick two fields per byte without normalising   (14 ops / 32 codes)
//   Q = 3, 4  : 2-bit then 4-bit fields, masks 0x0F / 0xF0                                       (23-24 ops)
//   Q = 5..8  : 2-, 4-, 8-bit fields, bytes come out normalised, one accumulator set             (<= 48 ops)
// against 16 Q ops for the plane-by-plane version (planes_to_bytes in abq_common.cuh).
#pragma once
#include <stdint.h>

namespace abq {

__device__ __forceinline__ uint32_t sel(uint32_t a, uint32_t b, uint32_t m) { return (a & m) | (b & ~m); }

// (p0, p1) -> 2-bit fields: lo has the fields of even bit positions, hi of odd bit positions
__device__ __forceinline__ void pair_fields(uint32_t p0, uint32_t p1, uint32_t &even, uint32_t &odd)
{
    even = sel(p0, p1 + p1, 0x55555555u);
    odd = sel(p0 >> 1, p1, 0x55555555u);
}

// four planes -> 4-bit fields: n[s] holds, in nibble c, the code of bit position 4c + s
__device__ __forceinline__ void nibble_fields(uint32_t p0, uint32_t p1, uint32_t p2, uint32_t p3, bool has_p3, uint32_t (&n)[4])
{
    uint32_t a0, a1, b0, b1;
    pair_fields(p0, p1, a0, a1);
    if (has_p3) {
        pair_fields(p2, p3, b0, b1);
    } else {
        b0 = p2 & 0x55555555u;
        b1 = (p2 >> 1) & 0x55555555u;
    }
    n[0] = sel(a0, b0 << 2, 0x33333333u);
    n[2] = sel(a0 >> 2, b0, 0x33333333u);
    n[1] = sel(a1, b1 << 2, 0x33333333u);
    n[3] = sel(a1 >> 2, b1, 0x33333333u);
}

template <int Q>
struct Expand {
    // Q = 5..8 (and the generic fallback): bytes come out normalised
    static constexpr int kSets = 1;
    static constexpr int kShift = 0;
    __device__ static constexpr int set_of_step(int) { return 0; }
    __device__ static __forceinline__ void run(const uint32_t (&p)[Q], uint32_t (&r)[8])
    {
        uint32_t lo[4], hi[4];
        nibble_fields(p[0], p[1], p[2], p[3], true, lo);
        const uint32_t p5 = Q > 5 ? p[Q > 5 ? 5 : 0] : 0u, p6 = Q > 6 ? p[Q > 6 ? 6 : 0] : 0u, p7 = Q > 7 ? p[Q > 7 ? 7 : 0] : 0u;
        nibble_fields(p[4], p5, p6, p7, Q > 7, hi);
#pragma unroll
        for (int s = 0; s < 4; ++s) {
            r[s] = sel(lo[s], hi[s] << 4, 0x0f0f0f0fu);
            r[4 + s] = sel(lo[s] >> 4, hi[s], 0x0f0f0f0fu);
        }
    }
};

template <>
struct Expand<1> {
    static constexpr int kSets = 1;
    static constexpr int kShift = 0;
    __device__ static constexpr int set_of_step(int) { return 0; }
    __device__ static __forceinline__ void run(const uint32_t (&p)[1], uint32_t (&r)[8])
    {
#pragma unroll
        for (int s = 0; s < 8; ++s)
            r[s] = (p[0] >> s) & 0x01010101u;
    }
};

template <>
struct Expand<2> {
    // steps 0 and 2 carry the codes themselves, steps 1 and 3 carry 4 x code
    static constexpr int kSets = 2;
    static constexpr int kShift = 2;
    __device__ static constexpr int set_of_step(int i) { return i & 1; }
    __device__ static __forceinline__ void run(const uint32_t (&p)[2], uint32_t (&r)[8])
    {
        uint32_t e, o;
        pair_fields(p[0], p[1], e, o);
        const uint32_t e4 = e >> 4, o4 = o >> 4;
        r[0] = e & 0x03030303u;
        r[1] = o & 0x03030303u;
        r[2] = e & 0x0c0c0c0cu;
        r[3] = o & 0x0c0c0c0cu;
        r[4] = e4 & 0x03030303u;
        r[5] = o4 & 0x03030303u;
        r[6] = e4 & 0x0c0c0c0cu;
        r[7] = o4 & 0x0c0c0c0cu;
    }
};

template <int Q>
struct ExpandNibble {
    // steps 0, 1 carry the codes, steps 2, 3 carry 16 x code
    static constexpr int kSets = 2;
    static constexpr int kShift = 4;
    __device__ static constexpr int set_of_step(int i) { return i >> 1; }
    __device__ static __forceinline__ void run(const uint32_t (&p)[Q], uint32_t (&r)[8])
    {
        uint32_t n[4];
        nibble_fields(p[0], p[1], p[2], Q > 3 ? p[Q > 3 ? 3 : 0] : 0u, Q > 3, n);
#pragma unroll
        for (int s = 0; s < 4; ++s) {
            r[s] = n[s] & 0x0f0f0f0fu;
            r[4 + s] = n[s] & 0xf0f0f0f0u;
        }
    }
};
template <>
struct Expand<3> : ExpandNibble<3> {};
template <>
struct Expand<4> : ExpandNibble<4> {};

} // namespace abq
