// Route A (ABQ_ROUTE_B1_MMA): the reference's formulation kept as a second, independent route --
// 1-bit tensor-core MMAs (mma.sync.m8n8k128 b1 AND+POPC) over pairs of bit-planes, combined by
// shift-accumulate with two's complement plane weights (engine/mma_any/aq_bmma_kernel.h:227-251,
// 537-565; PTX wrapper engine/mma_any/bmma.h:215).  sm_100a has no native 1-bit tensor path (the
// instruction is emulated, about 0.1 warp-MMA per ns per SM), so this route is a cross-check and a
// benchmark line, never the automatic choice.  One warp per 8 x 8 output tile, fragments loaded
// straight from global memory (the working set of a tile is L1/L2 resident).
#include "abq_common.cuh"
#include "abq_kernels.h"

namespace abq {

struct B1Args {
    int M, N, K;
    const uint32_t *X, *W;
    void *D;
    const __half *C;
    const __half *w_scale;
    const float *x_scale;
    int x_bits, w_bits, x_signed, w_signed;
    int out_dtype, scale_mode;
};

__device__ __forceinline__ void bmma_8x8x128(int (&d)[2], uint32_t a, uint32_t b)
{
    asm volatile("mma.sync.aligned.m8n8k128.row.col.s32.b1.b1.s32.and.popc {%0,%1}, {%2}, {%3}, {%0,%1};\n"
                 : "+r"(d[0]), "+r"(d[1])
                 : "r"(a), "r"(b));
}

__global__ void __launch_bounds__(128) b1_kernel(const B1Args a)
{
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = (blockIdx.x * 4 + warp) * 8;
    const int m0 = blockIdx.y * 8;
    if (n0 >= a.N)
        return;
    const int KW = a.K >> 5;
    const int r = lane >> 2, kq = lane & 3; // fragment row (token or weight row) and k word of this lane
    const int m = m0 + r, n = n0 + r;
    const bool mv = m < a.M, nv = n < a.N;
    const size_t xplane = (size_t)a.M * KW, wplane = (size_t)a.N * KW;
    int total[2] = { 0, 0 };
    for (int i = 0; i < a.x_bits; ++i) {
        int acc[8][2];
#pragma unroll
        for (int j = 0; j < 8; ++j)
            acc[j][0] = acc[j][1] = 0;
        const uint32_t *xp = a.X + i * xplane + (size_t)m * KW + kq;
        for (int ks = 0; ks < KW; ks += 4) {
            const uint32_t af = mv ? __ldg(xp + ks) : 0u;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                if (j < a.w_bits) {
                    const uint32_t bf = nv ? __ldg(a.W + j * wplane + (size_t)n * KW + kq + ks) : 0u;
                    bmma_8x8x128(acc[j], af, bf);
                }
            }
        }
        const int xmul = (a.x_signed && i == a.x_bits - 1) ? -(1 << i) : (1 << i);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            if (j < a.w_bits) {
                const int wmul = (a.w_signed && j == a.w_bits - 1) ? -(1 << j) : (1 << j);
                total[0] += xmul * wmul * acc[j][0];
                total[1] += xmul * wmul * acc[j][1];
            }
        }
    }
    // accumulator layout: token row = lane / 4, weight columns 2 * (lane % 4) and + 1
    const int tok = m0 + (lane >> 2);
#pragma unroll
    for (int e = 0; e < 2; ++e) {
        const int col = n0 + 2 * (lane & 3) + e;
        if (tok < a.M && col < a.N) {
            const size_t o = (size_t)tok * a.N + col;
            if (a.out_dtype == ABQ_OUT_INT32) {
                reinterpret_cast<int *>(a.D)[o] = total[e];
            } else if (a.scale_mode == ABQ_SCALE_TENSOR_COMPAT) {
                reinterpret_cast<__half *>(a.D)[o] = __hmul(__int2half_rn(total[e]), ld_half(a.C));
            } else {
                float v = (float)total[e] * __half2float(ld_half(a.w_scale + col));
                if (a.x_scale)
                    v *= __ldg(a.x_scale + tok);
                reinterpret_cast<__half *>(a.D)[o] = __float2half_rn(v);
            }
        }
    }
}

abq_status b1_plan(abq_gemm_state *st)
{
    const abq_gemm_params &p = st->p;
    if (p.scale_mode == ABQ_SCALE_GROUP || (p.scale_mode == ABQ_SCALE_CHANNEL && p.w_zero))
        return ABQ_ERR_UNSUPPORTED; // zero points / groups need the code sums only the int8 routes keep
    st->grid[0] = (p.N + 31) / 32;
    st->grid[1] = (p.M + 7) / 8;
    st->grid[2] = 1;
    st->block[0] = 128;
    st->block[1] = st->block[2] = 1;
    st->cluster = 1;
    st->shared_mem_size = 0;
    return ABQ_OK;
}

cudaError_t b1_launch(const abq_gemm_state *st, cudaStream_t stream)
{
    const abq_gemm_params &p = st->p;
    B1Args a;
    a.M = p.M;
    a.N = p.N;
    a.K = p.K;
    a.X = reinterpret_cast<const uint32_t *>(p.X);
    a.W = reinterpret_cast<const uint32_t *>(p.W);
    a.D = p.D;
    a.C = reinterpret_cast<const __half *>(p.C);
    a.w_scale = reinterpret_cast<const __half *>(p.w_scale);
    a.x_scale = p.x_scale;
    a.x_bits = p.x_bits;
    a.w_bits = p.w_bits;
    a.x_signed = p.x_signed;
    a.w_signed = p.w_signed;
    a.out_dtype = p.out_dtype;
    a.scale_mode = p.scale_mode;
    b1_kernel<<<dim3(st->grid[0], st->grid[1]), 128, 0, stream>>>(a);
    return cudaGetLastError();
}

} // namespace abq
