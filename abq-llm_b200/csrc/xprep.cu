// Plane -> byte expansion kernels that feed the integer tensor-core routes.
//
//  * unpack_i8:      planes[bits][rows][K/32] -> int8/uint8 codes [rows][K] (row-major, K contiguous);
//                    operand format of the tcgen05 route.  (The decode route expands its activation planes
//                    inside the GEMM kernel, see gemm_decode.cu.)
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

} // namespace abq
