// Route A (ABQ_ROUTE_B1_MMA): the reference's own formulation, kept as a second, independent route -- 1-bit tensor-core
// MMAs (mma.sync.m8n8k128 b1 AND+POPC) over pairs of bit-planes, combined by shift-accumulate with two's complement plane
// weights (engine/mma_any/aq_bmma_kernel.h:227-251, 537-565; PTX wrapper engine/mma_any/bmma.h:215).
//
// As there, the planes of an operand are stacked along its row dimension, so one 8 x 8 x 128 MMA multiplies eight
// (token, plane) rows by eight (weight row, plane) rows and no MMA row is wasted on a token that does not exist (one
// token with eight activation bits fills a tile by itself):
//   activations  stacked row sx = token * x_bits + plane            (token-major; tiles of 8 consecutive stacked rows)
//   weights      per warp 8 weight rows; tile j = plane j of them   (plane-major)
// A CTA of four warps owns 32 weight rows x BM tokens over all of K.  The operand bits travel global -> shared memory in
// 16-byte cp.async pieces (three stages of 1024 features; rows out of range and the K tail are zero-filled), XOR-swizzled
// so that the fragment reads of a warp touch 32 different banks.  Per 128 features a warp loads its SXT + Q fragments
// once and issues SXT * Q MMAs; the raw popcount sums stay in registers over the whole K loop (SXT * Q <= 32 tiles, which
// bounds the tokens per CTA: BM = floor(8 * SXT / x_bits)), then every lane adds its sums, shifted and signed, into the
// CTA's int32 output tile in shared memory, and the tile leaves through the epilogue of the requested mode.
// sm_100a has no native 1-bit tensor path (the instruction is emulated), so this route is a cross-check and a benchmark
// line, never the automatic choice.
#include "abq_common.cuh"
#include "abq_kernels.h"

namespace abq {

constexpr int kB1Warps = 4;
constexpr int kB1Threads = kB1Warps * 32;
constexpr int kB1BN = kB1Warps * 8;    // weight rows per CTA
constexpr int kB1StageWords = 32;      // 1024 features per stage and stacked row
constexpr int kB1Stages = 3;

struct B1Args {
    int M, N, K;
    const uint32_t *X, *W;
    void *D;
    const __half *C;
    const __half *w_scale;
    const float *x_scale;
    int x_bits, w_bits, x_signed, w_signed;
    int out_dtype, scale_mode;
    int bm; // tokens per CTA
};

__device__ __forceinline__ void bmma_8x8x128(int (&d)[2], uint32_t a, uint32_t b)
{
    asm volatile("mma.sync.aligned.m8n8k128.row.col.s32.b1.b1.s32.and.popc {%0,%1}, {%2}, {%3}, {%0,%1};\n"
                 : "+r"(d[0]), "+r"(d[1])
                 : "r"(a), "r"(b));
}

// 16 bytes global -> shared; `bytes` = 0 writes zeros without touching the source
__device__ __forceinline__ void cp_async_16(void *dst, const void *src, int bytes)
{
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(dst)), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// word w of stacked row r inside a stage: 16-byte pieces permuted by the row so that rows 0..7 x words c..c+3 are 32 banks
__device__ __forceinline__ int b1_swz(int r, int w) { return r * kB1StageWords + (w ^ ((r & 7) << 2)); }

template <int SXT, int Q>
__global__ void __launch_bounds__(kB1Threads) b1_kernel(const B1Args a)
{
    extern __shared__ __align__(16) uint32_t b1_smem[];
    constexpr int XR = SXT * 8;    // stacked activation rows of the CTA
    constexpr int WR = kB1BN * Q;  // stacked weight rows of the CTA: [warp][plane][8 rows]
    constexpr int kStage = (XR + WR) * kB1StageWords;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, kq = lane & 3;
    const int n0 = blockIdx.x * kB1BN, m0 = blockIdx.y * a.bm;
    const int KW = a.K >> 5;
    const int stages_total = (KW + kB1StageWords - 1) / kB1StageWords;
    const int live_sx = min(a.bm, a.M - m0) * a.x_bits; // stacked activation rows that exist

    auto fetch = [&](int stage) {
        uint32_t *dst = b1_smem + (size_t)(stage % kB1Stages) * kStage;
        const int kw0 = stage * kB1StageWords;
        for (int c = threadIdx.x; c < (XR + WR) * (kB1StageWords / 4); c += kB1Threads) {
            const int r = c / (kB1StageWords / 4), piece = c % (kB1StageWords / 4);
            const int kw = kw0 + piece * 4;
            const uint32_t *src = a.X;
            bool live = kw < KW;
            if (r < XR) {
                const int tok = r / a.x_bits, plane = r - tok * a.x_bits;
                live = live && r < live_sx;
                src = a.X + ((size_t)plane * a.M + (m0 + tok)) * KW + kw;
            } else {
                const int wr = r - XR, w = wr / (8 * Q), plane = (wr / 8) % Q, row = n0 + w * 8 + (wr & 7);
                live = live && row < a.N;
                src = a.W + ((size_t)plane * a.N + row) * KW + kw;
            }
            cp_async_16(dst + b1_swz(r, piece * 4), live ? src : a.X, live ? 16 : 0);
        }
        cp_async_commit();
    };

    int acc[SXT][Q][2];
#pragma unroll
    for (int s = 0; s < SXT; ++s)
#pragma unroll
        for (int j = 0; j < Q; ++j)
            acc[s][j][0] = acc[s][j][1] = 0;

    for (int s = 0; s < kB1Stages - 1; ++s) {
        if (s < stages_total)
            fetch(s);
        else
            cp_async_commit(); // keeps the group count in step
    }
    for (int st = 0; st < stages_total; ++st) {
        cp_async_wait<kB1Stages - 2>(); // the group of stage st has landed (for this thread)
        __syncthreads();                // ... for every thread; and stage st - 1 has been read by everybody
        if (st + kB1Stages - 1 < stages_total)
            fetch(st + kB1Stages - 1);  // into the buffer of stage st - 1
        else
            cp_async_commit();
        const uint32_t *xs = b1_smem + (size_t)(st % kB1Stages) * kStage;
        const uint32_t *ws = xs + XR * kB1StageWords + warp * (8 * Q) * kB1StageWords;
#pragma unroll
        for (int ks = 0; ks < kB1StageWords / 4; ++ks) {
            uint32_t af[SXT], bf[Q];
#pragma unroll
            for (int s = 0; s < SXT; ++s)
                af[s] = xs[b1_swz(s * 8 + g, ks * 4 + kq)];
#pragma unroll
            for (int j = 0; j < Q; ++j)
                bf[j] = ws[b1_swz(j * 8 + g, ks * 4 + kq)];
#pragma unroll
            for (int s = 0; s < SXT; ++s)
#pragma unroll
                for (int j = 0; j < Q; ++j)
                    bmma_8x8x128(acc[s][j], af[s], bf[j]);
        }
    }
    cp_async_wait<0>();
    __syncthreads(); // the stages are dead: their memory becomes the output tile

    // ---- shift-accumulate: acc[s][j][e] is the popcount sum of stacked activation row s * 8 + g and plane j of weight
    // row warp * 8 + 2 * kq + e
    int *tile = reinterpret_cast<int *>(b1_smem); // [bm][32]
    for (int i = threadIdx.x; i < a.bm * kB1BN; i += kB1Threads)
        tile[i] = 0;
    __syncthreads();
#pragma unroll
    for (int s = 0; s < SXT; ++s) {
        const int sx = s * 8 + g;
        if (sx < live_sx) {
            const int tok = sx / a.x_bits, xi = sx - tok * a.x_bits;
            const int xmul = (a.x_signed && xi == a.x_bits - 1) ? -(1 << xi) : (1 << xi);
            int sum[2] = { 0, 0 };
#pragma unroll
            for (int j = 0; j < Q; ++j) {
                const int wmul = (a.w_signed && j == Q - 1) ? -(1 << j) : (1 << j);
                sum[0] += wmul * acc[s][j][0];
                sum[1] += wmul * acc[s][j][1];
            }
            atomicAdd(&tile[tok * kB1BN + warp * 8 + 2 * kq], xmul * sum[0]);
            atomicAdd(&tile[tok * kB1BN + warp * 8 + 2 * kq + 1], xmul * sum[1]);
        }
    }
    __syncthreads();
    const int toks = min(a.bm, a.M - m0);
    for (int i = threadIdx.x; i < toks * kB1BN; i += kB1Threads) {
        const int tok = m0 + i / kB1BN, col = n0 + i % kB1BN;
        if (col >= a.N)
            continue;
        const int total = tile[i];
        const size_t o = (size_t)tok * a.N + col;
        if (a.out_dtype == ABQ_OUT_INT32) {
            reinterpret_cast<int *>(a.D)[o] = total;
        } else if (a.scale_mode == ABQ_SCALE_TENSOR_COMPAT) {
            reinterpret_cast<__half *>(a.D)[o] = __hmul(__int2half_rn(total), ld_half(a.C));
        } else {
            float v = (float)total * __half2float(ld_half(a.w_scale + col));
            if (a.x_scale)
                v *= __ldg(a.x_scale + tok);
            reinterpret_cast<__half *>(a.D)[o] = __float2half_rn(v);
        }
    }
}

namespace {

// activation tiles per CTA: the smallest power of two that holds all tokens' stacked rows, at most 32 / Q tiles (the raw
// sums of SXT * Q tiles live in registers) -- then halved while the launch would leave SMs with fewer than three CTAs
// (the emulated MMA needs many warps in flight; the weights a CTA re-reads come out of L2) and a token's planes still fit
int b1_tiles(int M, int N, int x_bits, int w_bits)
{
    int cap = 1;
    while (cap * 2 * w_bits <= 32)
        cap *= 2;
    int sxt = 1;
    while (sxt < cap && sxt * 8 < M * x_bits)
        sxt *= 2;
    int sms = 148, dev = 0, v = 0;
    if (cudaGetDevice(&dev) == cudaSuccess && cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && v > 0)
        sms = v;
    const long col_ctas = (N + kB1BN - 1) / kB1BN;
    while (sxt > 1 && (sxt / 2) * 8 >= x_bits) {
        const int bm = sxt * 8 / x_bits;
        if (col_ctas * ((M + bm - 1) / bm) >= 3L * sms)
            break;
        sxt /= 2;
    }
    return sxt;
}

size_t b1_smem_bytes(int sxt, int q, int bm)
{
    const size_t stages = (size_t)kB1Stages * (sxt * 8 + kB1BN * q) * kB1StageWords * 4;
    const size_t tile = (size_t)bm * kB1BN * 4;
    return stages > tile ? stages : tile;
}

template <int SXT, int Q>
cudaError_t b1_launch_variant(const B1Args &a, dim3 grid, size_t smem, cudaStream_t stream)
{
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(b1_kernel<SXT, Q>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess)
            return e;
    }
    b1_kernel<SXT, Q><<<grid, kB1Threads, smem, stream>>>(a);
    return cudaGetLastError();
}

template <int Q>
cudaError_t b1_launch_q(int sxt, const B1Args &a, dim3 grid, size_t smem, cudaStream_t stream)
{
    switch (sxt) {
    case 1: return b1_launch_variant<1, Q>(a, grid, smem, stream);
    case 2: return b1_launch_variant<2, Q>(a, grid, smem, stream);
    case 4: return b1_launch_variant<4, Q>(a, grid, smem, stream);
    case 8:
        if constexpr (8 * Q <= 32)
            return b1_launch_variant<8, Q>(a, grid, smem, stream);
        break;
    case 16:
        if constexpr (16 * Q <= 32)
            return b1_launch_variant<16, Q>(a, grid, smem, stream);
        break;
    case 32:
        if constexpr (32 * Q <= 32)
            return b1_launch_variant<32, Q>(a, grid, smem, stream);
        break;
    }
    return cudaErrorInvalidValue;
}

} // namespace

abq_status b1_plan(abq_gemm_state *st)
{
    const abq_gemm_params &p = st->p;
    if (p.scale_mode == ABQ_SCALE_GROUP || (p.scale_mode == ABQ_SCALE_CHANNEL && p.w_zero))
        return ABQ_ERR_UNSUPPORTED; // zero points / groups need the code sums only the int8 routes keep
    const int sxt = b1_tiles(p.M, p.N, p.x_bits, p.w_bits);
    const int bm = sxt * 8 / p.x_bits; // >= 1: a tile holds the eight planes of a token at most
    st->grid[0] = (p.N + kB1BN - 1) / kB1BN;
    st->grid[1] = (p.M + bm - 1) / bm;
    st->grid[2] = 1;
    st->block[0] = kB1Threads;
    st->block[1] = st->block[2] = 1;
    st->cluster = 1;
    st->shared_mem_size = b1_smem_bytes(sxt, p.w_bits, bm);
    st->tile[0] = sxt;
    st->tile[1] = bm;
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
    a.bm = st->tile[1];
    const dim3 grid(st->grid[0], st->grid[1]);
    const int sxt = st->tile[0];
    switch (p.w_bits) {
    case 1: return b1_launch_q<1>(sxt, a, grid, st->shared_mem_size, stream);
    case 2: return b1_launch_q<2>(sxt, a, grid, st->shared_mem_size, stream);
    case 3: return b1_launch_q<3>(sxt, a, grid, st->shared_mem_size, stream);
    case 4: return b1_launch_q<4>(sxt, a, grid, st->shared_mem_size, stream);
    case 5: return b1_launch_q<5>(sxt, a, grid, st->shared_mem_size, stream);
    case 6: return b1_launch_q<6>(sxt, a, grid, st->shared_mem_size, stream);
    case 7: return b1_launch_q<7>(sxt, a, grid, st->shared_mem_size, stream);
    case 8: return b1_launch_q<8>(sxt, a, grid, st->shared_mem_size, stream);
    }
    return cudaErrorInvalidValue;
}

} // namespace abq
