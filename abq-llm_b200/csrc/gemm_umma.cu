// Prefill-shape GEMM (M > 16), route ABQ_ROUTE_I8_UMMA ("route B").
//
// tcgen05 has no 1-bit MMA kind, but integer arithmetic is exact and associative, so the shift-accumulate
// over plane pairs (engine/mma_any/aq_bmma_kernel.h:537-565) can be folded into the operands: the p (q) planes
// of an operand are recombined once into 8-bit codes (unpack_i8, xprep.cu) and ONE tcgen05.mma kind::i8 per
// 128 x BN x 32 block replaces the p*q plane-pair MMAs, with a bit-identical int32 result
// (|acc| <= 255 * 255 * K < 2^31 for K <= 33 000).
//
// Kernel: one CTA per 128 x BN output tile.
//   warp 0      TMA producer: A (activations, 128 rows x 128 B) and B (weights, BN rows x 128 B) tiles of a
//               K block into a ring of 128B-swizzled stages, completion on mbarriers
//   warp 1      allocates TMEM, one elected thread issues four 128 x BN x 32 UMMAs per stage (smem descriptors
//               advanced by 32 B inside the swizzle atom), tcgen05.commit frees the stage / signals the epilogue
//   warps 2..5  epilogue: tcgen05.ld the int32 accumulators (lane = output row), fused dequantisation, stores
// Every wait is bounded (abq_common.cuh); on expiry the status word is set, the roles leave their loops, the
// CTA still meets at the final barrier and TMEM is released.
#include <cuda.h>
#include <cstring>

#include "abq_common.cuh"
#include "abq_kernels.h"

namespace abq {

constexpr int kUmmaThreads = 192;
constexpr int kUmmaBM = 128;
constexpr int kUmmaBK = 128; // bytes (= int8 elements) per stage along K: one 128B swizzle atom row

struct UmmaArgs {
    int M, N, K;
    int stages;
    void *D;
    const __half *C;
    const __half *w_scale;
    const uint8_t *w_zero;
    const float *x_scale;
    const int *xsum; // per-token code sums (only with zero points)
    int out_dtype, scale_mode;
    uint32_t idesc;
    int *status;
};

__device__ __forceinline__ uint64_t make_smem_desc_sw128(uint32_t smem_addr)
{
    // K-major operand tile, 128-byte rows, SWIZZLE_128B: 8-row groups are 1024 B apart (stride byte offset);
    // the leading byte offset is not used for swizzled K-major layouts (encoded as 1); descriptor version 1.
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3ffff) >> 4);       // start address, 16-byte units, bits [0,14)
    d |= (uint64_t)1 << 16;                            // leading byte offset (16 B units), bits [16,30)
    d |= (uint64_t)(1024 >> 4) << 32;                  // stride byte offset (16 B units), bits [32,46)
    d |= (uint64_t)1 << 46;                            // version (Blackwell), bits [46,48)
    d |= (uint64_t)2 << 61;                            // layout type SWIZZLE_128B, bits [61,64)
    return d;
}

__device__ __forceinline__ void umma_i8(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate)
{
    asm volatile("{\n"
                 ".reg .pred p;\n"
                 "setp.ne.b32 p, %4, 0;\n"
                 "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n"
                 "}\n" ::"r"(tmem_d),
                 "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
                 : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t *bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// 32 consecutive accumulator columns of this thread's TMEM lane
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, int (&v)[32])
{
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                 "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]),
                   "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]),
                   "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]),
                   "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
                 : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

template <int BN>
__global__ void __launch_bounds__(kUmmaThreads, 1) umma_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                                                               const UmmaArgs a)
{
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    constexpr int kABytes = kUmmaBM * kUmmaBK, kBBytes = BN * kUmmaBK, kStageBytes = kABytes + kBBytes;
    constexpr int kTmemCols = BN < 32 ? 32 : BN; // power of two >= 32
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + (size_t)a.stages * kStageBytes);
    uint64_t *full = bars, *empty = bars + 8, *acc_full = bars + 16;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 17);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m0 = blockIdx.y * kUmmaBM, n0 = blockIdx.x * BN;
    const int k_blocks = a.K / kUmmaBK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < a.stages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        mbar_init(acc_full, 1);
        fence_mbar_init();
        prefetch_tmap(&tmap_a);
        prefetch_tmap(&tmap_b);
    }
    if (warp == 1) { // TMEM allocation is a warp-wide operation; the same warp frees it at the end
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tmem_fence_before();
    __syncthreads();
    tmem_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            for (int kb = 0; kb < k_blocks; ++kb) {
                const int s = kb % a.stages;
                if (kb >= a.stages && !mbar_wait_bounded(&empty[s], ((kb / a.stages) - 1) & 1, a.status, STATUS_TIMEOUT_PIPE))
                    break;
                uint8_t *sa = smem + (size_t)s * kStageBytes, *sb = sa + kABytes;
                mbar_arrive_expect_tx(&full[s], kStageBytes);
                tma_load_2d(sa, &tmap_a, kb * kUmmaBK, m0, &full[s]);
                tma_load_2d(sb, &tmap_b, kb * kUmmaBK, n0, &full[s]);
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        if (lane == 0) {
            bool ok = true;
            for (int kb = 0; kb < k_blocks && ok; ++kb) {
                const int s = kb % a.stages;
                ok = mbar_wait_bounded(&full[s], (kb / a.stages) & 1, a.status, STATUS_TIMEOUT_TMA);
                if (!ok)
                    break;
                tmem_fence_after();
                const uint32_t sa = smem_u32(smem + (size_t)s * kStageBytes), sb = sa + kABytes;
                const uint64_t da = make_smem_desc_sw128(sa), db = make_smem_desc_sw128(sb);
#pragma unroll
                for (int k = 0; k < kUmmaBK / 32; ++k) // 32 bytes of K per instruction: advance the start address inside the atom
                    umma_i8(tmem_base, da + (uint64_t)(k * 32 >> 4), db + (uint64_t)(k * 32 >> 4), a.idesc, (kb | k) != 0);
                umma_commit(&empty[s]); // arrives when the MMAs above have finished reading this stage
            }
            umma_commit(acc_full); // arrives when all MMAs have written the accumulator
        }
        __syncwarp();
    } else {
        // epilogue warps 2..5: a warp may only touch the TMEM lane quarter (warp id % 4)
        const int quarter = warp & 3;
        const int row = m0 + quarter * 32 + lane;
        const bool ok = mbar_wait_bounded(acc_full, 0, a.status, STATUS_TIMEOUT_MMA);
        tmem_fence_after();
        if (ok) {
            float xs = 1.f;
            int xsum = 0;
            if (row < a.M) {
                if (a.x_scale)
                    xs = a.x_scale[row];
                if (a.xsum)
                    xsum = a.xsum[row];
            }
            const __half cscale = a.scale_mode == ABQ_SCALE_TENSOR_COMPAT ? ld_half(a.C) : __half();
#pragma unroll 1
            for (int c = 0; c < BN; c += 32) {
                int v[32];
                tmem_ld32(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)c, v);
                if (row >= a.M)
                    continue;
                const int nb = n0 + c;
                if (a.out_dtype == ABQ_OUT_INT32) {
                    int *dst = reinterpret_cast<int *>(a.D) + (size_t)row * a.N + nb;
                    if (nb + 32 <= a.N && (a.N & 3) == 0) {
#pragma unroll
                        for (int j = 0; j < 32; j += 4)
                            *reinterpret_cast<int4 *>(dst + j) = make_int4(v[j], v[j + 1], v[j + 2], v[j + 3]);
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            if (nb + j < a.N)
                                dst[j] = v[j];
                    }
                } else {
                    __half h[32];
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        const int n = nb + j;
                        if (a.scale_mode == ABQ_SCALE_TENSOR_COMPAT) {
                            h[j] = __hmul(__int2half_rn(v[j]), cscale);
                        } else {
                            float f = 0.f;
                            if (n < a.N) {
                                int x = v[j];
                                if (a.w_zero)
                                    x -= (int)a.w_zero[n] * xsum;
                                f = (float)x * __half2float(ld_half(a.w_scale + n)) * xs;
                            }
                            h[j] = __float2half_rn(f);
                        }
                    }
                    __half *dst = reinterpret_cast<__half *>(a.D) + (size_t)row * a.N + nb;
                    if (nb + 32 <= a.N && (a.N & 7) == 0) {
#pragma unroll
                        for (int j = 0; j < 32; j += 8)
                            *reinterpret_cast<uint4 *>(dst + j) = *reinterpret_cast<const uint4 *>(&h[j]);
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            if (nb + j < a.N)
                                dst[j] = h[j];
                    }
                }
            }
        }
    }

    tmem_fence_before();
    __syncthreads();
    if (warp == 1) {
        tmem_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    }
}

// per-token sum of the int8 / uint8 activation codes (needed only with weight zero points)
__global__ void __launch_bounds__(256) rowsum_kernel(const uint8_t *__restrict__ x, int *__restrict__ out, int M, int K, int is_signed)
{
    const int row = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (row >= M)
        return;
    const uint32_t *p = reinterpret_cast<const uint32_t *>(x + (size_t)row * K);
    int s = 0;
    for (int i = lane; i < K / 4; i += 32) {
        const uint32_t w = __ldg(p + i);
        s = is_signed ? __dp4a((int)w, 0x01010101, s) : (int)__dp4a(w, 0x01010101u, (unsigned)s);
    }
#pragma unroll
    for (int o = 16; o; o >>= 1)
        s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0)
        out[row] = s;
}

// ------------------------------------------------------------------------------------------- host side

// workspace: [X codes M x K][W codes N x K][token sums M]
static void umma_layout(int M, int N, int K, size_t *off_w, size_t *off_sum, size_t *total)
{
    *off_w = ((size_t)M * K + 255) & ~(size_t)255;
    *off_sum = (*off_w + (size_t)N * K + 255) & ~(size_t)255;
    *total = *off_sum + (size_t)M * 4;
}

size_t umma_workspace_bytes(int M, int N, int K)
{
    size_t a, b, t;
    umma_layout(M, N, K, &a, &b, &t);
    return t;
}

abq_status umma_plan(abq_gemm_state *st)
{
    const abq_gemm_params &p = st->p;
    if (p.scale_mode == ABQ_SCALE_GROUP)
        return ABQ_ERR_UNSUPPORTED; // per-group scales need the accumulator drained per group: decode route only so far
    size_t off_w, off_sum, total;
    umma_layout(p.M, p.N, p.K, &off_w, &off_sum, &total);
    if (!p.workspace || p.workspace_bytes < total)
        return ABQ_ERR_WORKSPACE;
    if (reinterpret_cast<uintptr_t>(p.workspace) & 255)
        return ABQ_ERR_INVALID_ARG;
    int sms = 148;
    {
        int dev = 0, v = 0;
        if (cudaGetDevice(&dev) == cudaSuccess && cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && v > 0)
            sms = v;
    }
    // widest N tile that still gives every SM a CTA
    const int m_tiles = (p.M + kUmmaBM - 1) / kUmmaBM;
    int BN = 256;
    while (BN > 64 && (long)m_tiles * ((p.N + BN - 1) / BN) < sms)
        BN >>= 1;
    BN = env_int("ABQ_UMMA_BN", BN);
    if (BN != 64 && BN != 128 && BN != 256)
        return ABQ_ERR_INVALID_ARG;
    const int stage_bytes = (kUmmaBM + BN) * kUmmaBK;
    int stages = (200 * 1024) / stage_bytes;
    stages = stages > 8 ? 8 : stages;
    const int k_blocks = p.K / kUmmaBK;
    stages = stages > k_blocks ? k_blocks : stages;
    stages = env_int("ABQ_UMMA_STAGES", stages);
    if (stages < 1 || stages > 8)
        return ABQ_ERR_INVALID_ARG;

    uint8_t *ws = reinterpret_cast<uint8_t *>(p.workspace);
    const uint64_t dims_a[2] = { (uint64_t)p.K, (uint64_t)p.M }, dims_b[2] = { (uint64_t)p.K, (uint64_t)p.N };
    const uint64_t strides[1] = { (uint64_t)p.K };
    const uint32_t box_a[2] = { (uint32_t)kUmmaBK, (uint32_t)kUmmaBM }, box_b[2] = { (uint32_t)kUmmaBK, (uint32_t)BN };
    if (!encode_tmap(st->tmap[0], TMAP_U8, 2, ws, dims_a, strides, box_a, TMAP_SWIZZLE_128B) ||
        !encode_tmap(st->tmap[1], TMAP_U8, 2, ws + off_w, dims_b, strides, box_b, TMAP_SWIZZLE_128B))
        return ABQ_ERR_CUDA;
    st->grid[0] = (p.N + BN - 1) / BN;
    st->grid[1] = m_tiles;
    st->grid[2] = 1;
    st->block[0] = kUmmaThreads;
    st->block[1] = st->block[2] = 1;
    st->cluster = 1;
    st->shared_mem_size = 1024 + (size_t)stages * stage_bytes + 256;
    st->tile[0] = BN;
    st->tile[1] = stages;
    return ABQ_OK;
}

template <int BN>
static cudaError_t launch_bn(const abq_gemm_state *st, const UmmaArgs &args, cudaStream_t stream)
{
    auto kern = umma_kernel<BN>;
    static thread_local size_t configured = 0;
    if (st->shared_mem_size > configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)st->shared_mem_size);
        if (e != cudaSuccess)
            return e;
        configured = st->shared_mem_size;
    }
    CUtensorMap ta, tb;
    memcpy(&ta, st->tmap[0], sizeof(ta));
    memcpy(&tb, st->tmap[1], sizeof(tb));
    kern<<<dim3(st->grid[0], st->grid[1]), kUmmaThreads, st->shared_mem_size, stream>>>(ta, tb, args);
    return cudaGetLastError();
}

cudaError_t umma_launch(const abq_gemm_state *st, cudaStream_t stream)
{
    const abq_gemm_params &p = st->p;
    size_t off_w, off_sum, total;
    umma_layout(p.M, p.N, p.K, &off_w, &off_sum, &total);
    uint8_t *ws = reinterpret_cast<uint8_t *>(p.workspace);
    cudaError_t e = unpack_i8(reinterpret_cast<const uint32_t *>(p.X), ws, p.M, p.K, p.x_bits, p.x_signed, stream);
    if (e != cudaSuccess)
        return e;
    e = unpack_i8(reinterpret_cast<const uint32_t *>(p.W), ws + off_w, p.N, p.K, p.w_bits, p.w_signed, stream);
    if (e != cudaSuccess)
        return e;
    UmmaArgs a;
    a.xsum = nullptr;
    if (p.scale_mode == ABQ_SCALE_CHANNEL && p.w_zero) {
        rowsum_kernel<<<(p.M + 7) / 8, 256, 0, stream>>>(ws, reinterpret_cast<int *>(ws + off_sum), p.M, p.K, p.x_signed);
        e = cudaGetLastError();
        if (e != cudaSuccess)
            return e;
        a.xsum = reinterpret_cast<const int *>(ws + off_sum);
    }
    a.M = p.M;
    a.N = p.N;
    a.K = p.K;
    a.stages = st->tile[1];
    a.D = p.D;
    a.C = reinterpret_cast<const __half *>(p.C);
    a.w_scale = reinterpret_cast<const __half *>(p.w_scale);
    a.w_zero = p.w_zero;
    a.x_scale = p.x_scale;
    a.out_dtype = p.out_dtype;
    a.scale_mode = p.scale_mode;
    const int BN = st->tile[0];
    // instruction descriptor, kind::i8: D format S32 (2) at bit 4, A / B format (0 = U8, 1 = S8) at bits 7 / 10,
    // both operands K-major (bits 15, 16 clear), N >> 3 at bit 17, M >> 4 at bit 24
    a.idesc = (2u << 4) | ((p.x_signed ? 1u : 0u) << 7) | ((p.w_signed ? 1u : 0u) << 10) | ((uint32_t)(BN >> 3) << 17) |
              ((uint32_t)(kUmmaBM >> 4) << 24);
    a.status = p.status_word;
    switch (BN) {
    case 64: return launch_bn<64>(st, a, stream);
    case 128: return launch_bn<128>(st, a, stream);
    default: return launch_bn<256>(st, a, stream);
    }
}

} // namespace abq
