// Prefill-shape GEMM (more than 32 rows by default), route ABQ_ROUTE_I8_UMMA ("route B").
//
// tcgen05 has no 1-bit MMA kind, but integer arithmetic is exact and associative, so the shift-accumulate
// over plane pairs (engine/mma_any/aq_bmma_kernel.h:537-565) can be folded into the operands: the p (q) planes
// of an operand are recombined once into 8-bit codes (unpack_i8, xprep.cu) and ONE tcgen05.mma kind::i8 per
// 128 x BN x 32 block replaces the p*q plane-pair MMAs, with a bit-identical int32 result
// (|acc| <= 255 * 255 * K < 2^31 for K <= 33 000).
//
// Kernel: persistent, one CTA per SM, 128 x BN output tiles dealt round-robin (consecutive tiles share a weight tile).
//   warp 0      TMA producer: A (activations, 128 rows x 128 B) and B (weights, BN rows x 128 B) tiles of a
//               K block into a ring of 128B-swizzled stages that runs on across tile boundaries
//   warp 1      allocates TMEM (two accumulators of BN columns); one elected thread issues four 128 x BN x 32 UMMAs
//               per stage (smem descriptors advanced by 32 B inside the swizzle atom); tcgen05.commit frees the
//               stage and, after the last K block, hands the accumulator to the epilogue
//   warps 2..5  epilogue of the previous tile while the next one is being multiplied: channel scales / zero
//               points staged in shared memory, tcgen05.ld of the int32 accumulators (lane = output row), fused
//               dequantisation, 16-byte stores; then the accumulator goes back to the MMA warp
// Every wait is bounded (abq_common.cuh); on expiry the status word is set, the roles leave their loops, the
// CTA still meets at the final barrier and TMEM is released.
// Per-group scales: umma_group_kernel below (accumulator drained per scale group).
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
    const int *xsum; // per-token code sums (only with per-channel zero points)
    int kb_per_group;  // ABQ_SCALE_GROUP: 128-byte K blocks per scale group; 0: groups of 64 features, two per K block
    int scale_groups;  // ABQ_SCALE_GROUP: scale groups per weight row
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

// Epilogue of 32 accumulator columns of one output row.  MODE 0: int32, 1: fp16 times one fp16 factor (the
// reference's arithmetic: the accumulator rounded to fp16, then an fp16 multiply), 2: per-channel scale (and zero
// point) from shared memory, per-token scale from a register.
template <int MODE>
__device__ __forceinline__ void store_chunk(const UmmaArgs &a, const int (&v)[32], int row, int nb, const float *s_scale, const int *s_zero,
                                            float xs, int xsum, __half cscale, bool has_zero)
{
    if (MODE == 0) {
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
        return;
    }
    uint32_t h[16]; // 32 fp16 values, two per register
#pragma unroll
    for (int j = 0; j < 32; j += 4) {
        float f[4];
        if (MODE == 1) {
#pragma unroll
            for (int e = 0; e < 4; ++e)
                f[e] = 0.f;
            const __half2 c2 = __half2half2(cscale);
            const __half2 lo = __hmul2(__halves2half2(__int2half_rn(v[j]), __int2half_rn(v[j + 1])), c2);
            const __half2 hi = __hmul2(__halves2half2(__int2half_rn(v[j + 2]), __int2half_rn(v[j + 3])), c2);
            h[j / 2] = *reinterpret_cast<const uint32_t *>(&lo);
            h[j / 2 + 1] = *reinterpret_cast<const uint32_t *>(&hi);
        } else {
            const float4 sc = *reinterpret_cast<const float4 *>(s_scale + j); // same address in every lane: a broadcast
            int x[4] = { v[j], v[j + 1], v[j + 2], v[j + 3] };
            if (has_zero) {
                const int4 z = *reinterpret_cast<const int4 *>(s_zero + j);
                x[0] -= z.x * xsum;
                x[1] -= z.y * xsum;
                x[2] -= z.z * xsum;
                x[3] -= z.w * xsum;
            }
            f[0] = (float)x[0] * sc.x * xs; // same order of roundings as the reference-side formula: (acc * scale) * x_scale
            f[1] = (float)x[1] * sc.y * xs;
            f[2] = (float)x[2] * sc.z * xs;
            f[3] = (float)x[3] * sc.w * xs;
            const __half2 lo = __floats2half2_rn(f[0], f[1]), hi = __floats2half2_rn(f[2], f[3]);
            h[j / 2] = *reinterpret_cast<const uint32_t *>(&lo);
            h[j / 2 + 1] = *reinterpret_cast<const uint32_t *>(&hi);
        }
    }
    __half *dst = reinterpret_cast<__half *>(a.D) + (size_t)row * a.N + nb;
    if (nb + 32 <= a.N && (a.N & 7) == 0) {
#pragma unroll
        for (int j = 0; j < 16; j += 4)
            *reinterpret_cast<uint4 *>(dst + 2 * j) = make_uint4(h[j], h[j + 1], h[j + 2], h[j + 3]);
    } else {
#pragma unroll
        for (int j = 0; j < 32; ++j)
            if (nb + j < a.N)
                dst[j] = __ushort_as_half((unsigned short)(h[j >> 1] >> ((j & 1) * 16)));
    }
}

// the same without the wait: several loads in flight, then one tmem_ld_wait()
__device__ __forceinline__ void tmem_ld32_nowait(uint32_t taddr, int (&v)[32])
{
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                 "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]),
                   "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]),
                   "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]),
                   "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
                 : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

template <int BN>
__global__ void __launch_bounds__(kUmmaThreads, 1) umma_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                                                               const UmmaArgs a)
{
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    constexpr int kABytes = kUmmaBM * kUmmaBK, kBBytes = BN * kUmmaBK, kStageBytes = kABytes + kBBytes;
    constexpr int kTmemCols = 2 * BN; // two accumulators: the epilogue drains one while the next tile fills the other
    // 1024-byte alignment as an offset from the array itself: a pointer rebuilt from an integer would lose its address space
    // and every access behind it would compile to a generic load
    uint8_t *smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    float *s_scale = reinterpret_cast<float *>(smem + (size_t)a.stages * kStageBytes); // [2][BN] channel scales of a tile
    int *s_zero = reinterpret_cast<int *>(s_scale + 2 * BN);                            // [2][BN] channel zero points
    uint64_t *bars = reinterpret_cast<uint64_t *>(s_zero + 2 * BN);
    uint64_t *full = bars, *empty = bars + 8, *acc_full = bars + 16, *acc_empty = bars + 18, *par_ready = bars + 20;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 22);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int k_blocks = a.K / kUmmaBK;
    const int m_tiles = (a.M + kUmmaBM - 1) / kUmmaBM;
    const int total_tiles = m_tiles * ((a.N + BN - 1) / BN);

    if (threadIdx.x == 0) {
        for (int s = 0; s < a.stages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&acc_full[b], 1);
            mbar_init(&acc_empty[b], 4);    // one arrival per epilogue warp
            mbar_init(&par_ready[b], 128);  // every epilogue thread has staged its channel parameters
        }
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
    pdl_wait_prior_grid(); // operand codes and token sums come from the kernels launched just before

    // Persistent CTA: tiles blockIdx.x, blockIdx.x + gridDim.x, ...; consecutive tiles share the weight (N) tile, so
    // the CTAs running at one time read few distinct weight tiles and all of the activations out of L2.
    if (warp == 0) {
        if (lane == 0) {
            int kc = 0; // k-blocks requested so far, over all tiles
            bool ok = true;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
                const int m0 = (tile % m_tiles) * kUmmaBM, n0 = (tile / m_tiles) * BN;
                for (int kb = 0; kb < k_blocks; ++kb, ++kc) {
                    const int s = kc % a.stages;
                    if (kc >= a.stages && !mbar_wait_bounded(&empty[s], ((kc / a.stages) - 1) & 1, a.status, STATUS_TIMEOUT_PIPE)) {
                        ok = false;
                        break;
                    }
                    uint8_t *sa = smem + (size_t)s * kStageBytes, *sb = sa + kABytes;
                    mbar_arrive_expect_tx(&full[s], kStageBytes);
                    tma_load_2d(sa, &tmap_a, kb * kUmmaBK, m0, &full[s]);
                    tma_load_2d(sb, &tmap_b, kb * kUmmaBK, n0, &full[s]);
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        if (lane == 0) {
            int kc = 0, it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++it) {
                const int b = it & 1;
                if (it >= 2) { // the epilogue has drained this accumulator's previous tile
                    ok = mbar_wait_bounded(&acc_empty[b], ((it >> 1) - 1) & 1, a.status, STATUS_TIMEOUT_PIPE);
                    if (!ok)
                        break;
                    tmem_fence_after();
                }
                const uint32_t tmem_d = tmem_base + (uint32_t)(b * BN);
                for (int kb = 0; kb < k_blocks; ++kb, ++kc) {
                    const int s = kc % a.stages;
                    ok = mbar_wait_bounded(&full[s], (kc / a.stages) & 1, a.status, STATUS_TIMEOUT_TMA);
                    if (!ok)
                        break;
                    tmem_fence_after();
                    const uint32_t sa = smem_u32(smem + (size_t)s * kStageBytes), sb = sa + kABytes;
                    const uint64_t da = make_smem_desc_sw128(sa), db = make_smem_desc_sw128(sb);
#pragma unroll
                    for (int k = 0; k < kUmmaBK / 32; ++k) // 32 bytes of K per instruction: advance the start address inside the atom
                        umma_i8(tmem_d, da + (uint64_t)(k * 32 >> 4), db + (uint64_t)(k * 32 >> 4), a.idesc, (kb | k) != 0);
                    umma_commit(&empty[s]); // arrives when the MMAs above have finished reading this stage
                }
                if (ok)
                    umma_commit(&acc_full[b]); // arrives when all MMAs of the tile have written the accumulator
            }
        }
        __syncwarp();
    } else {
        // epilogue warps 2..5: a warp may only touch the TMEM lane quarter (warp id % 4)
        const int quarter = warp & 3;
        const int et = threadIdx.x - 64; // 0..127 among the epilogue threads
        const bool channel = a.out_dtype != ABQ_OUT_INT32 && a.scale_mode != ABQ_SCALE_TENSOR_COMPAT;
        const bool has_zero = channel && a.scale_mode == ABQ_SCALE_CHANNEL && a.w_zero != nullptr;
        const __half cscale = a.scale_mode == ABQ_SCALE_TENSOR_COMPAT && a.out_dtype != ABQ_OUT_INT32 ? ld_half(a.C) : __half();
        int it = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++it) {
            const int b = it & 1;
            const int m0 = (tile % m_tiles) * kUmmaBM, n0 = (tile / m_tiles) * BN;
            const int row = m0 + quarter * 32 + lane;
            float *ts = s_scale + b * BN;
            int *tz = s_zero + b * BN;
            if (channel) { // stage the tile's channel parameters while its MMAs still run
                for (int c = et; c < BN; c += 128) {
                    const int n = n0 + c;
                    float sv = 1.f;
                    int zv = 0;
                    if (n < a.N) {
                        if (a.scale_mode == ABQ_SCALE_CHANNEL && a.w_scale)
                            sv = __half2float(a.w_scale[n]);
                        if (has_zero)
                            zv = a.w_zero[n];
                    }
                    ts[c] = sv;
                    tz[c] = zv;
                }
                // epilogue threads only, and bounded like every other wait; the other buffer (tile it - 1) stays untouched
                mbar_arrive(&par_ready[b]);
                ok = mbar_wait_bounded(&par_ready[b], (it >> 1) & 1, a.status, STATUS_TIMEOUT_PIPE);
                if (!ok)
                    break;
            }
            float xs = 1.f;
            int xsum = 0;
            if (row < a.M) {
                if (a.x_scale)
                    xs = a.x_scale[row];
                if (a.xsum)
                    xsum = a.xsum[row];
            }
            ok = mbar_wait_bounded(&acc_full[b], (it >> 1) & 1, a.status, STATUS_TIMEOUT_MMA);
            if (!ok)
                break;
            tmem_fence_after();
#pragma unroll 1
            for (int c = 0; c < BN; c += 32) {
                int v[32];
                tmem_ld32(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(b * BN + c), v);
                if (row >= a.M)
                    continue;
                if (a.out_dtype == ABQ_OUT_INT32)
                    store_chunk<0>(a, v, row, n0 + c, ts + c, tz + c, xs, xsum, cscale, has_zero);
                else if (!channel)
                    store_chunk<1>(a, v, row, n0 + c, ts + c, tz + c, xs, xsum, cscale, has_zero);
                else
                    store_chunk<2>(a, v, row, n0 + c, ts + c, tz + c, xs, xsum, cscale, has_zero);
            }
            tmem_fence_before();
            __syncwarp();
            if (lane == 0)
                mbar_arrive(&acc_empty[b]); // this warp's quarter of the accumulator is free again
        }
    }

    tmem_fence_before();
    __syncthreads();
    if (warp == 1) {
        tmem_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    }
}

// ---------------------------------------------------------------------------------------------------------------
// ABQ_SCALE_GROUP on the tensor-core route: every scale group (kb_per_group K blocks) is multiplied into a fresh TMEM
// accumulator, exactly, and the epilogue warps drain it while the next group is multiplied into the other one:
//     facc[n] += scale[n][g] * acc_g[n]                                              (fp32, one row per thread)
// The zero points are not seen here: the weight codes in the scratch are w - zero[n][g] (signed int8, exact for widths
// up to 7 bits; see unpack_i8), so acc_g already is sum x * (w - z).  BN = 128 columns (128 fp32 partial sums per
// thread); the scales of the tile, all groups, are staged once per tile in shared memory as fp32 [group][column].
// MAGIC: |acc_g| < 2^22 (signed 8-bit activations, one K block per group): int -> float by the 1.5 * 2^23 trick, two
// pipelined operations instead of a conversion instruction.  Same roles, barriers and bounded waits as umma_kernel.
// cta_group::2 forms: issued by one thread of the even CTA of a pair
__device__ __forceinline__ void umma2_i8(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate)
{
    asm volatile("{\n"
                 ".reg .pred p;\n"
                 "setp.ne.b32 p, %4, 0;\n"
                 "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n"
                 "}\n" ::"r"(tmem_d),
                 "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
                 : "memory");
}
// arrives on the barrier at this shared-memory offset in both CTAs of the pair
__device__ __forceinline__ void umma2_commit(uint64_t *bar)
{
    const unsigned short both = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(smem_u32(bar)),
                 "h"(both)
                 : "memory");
}
// TMA tile load into this CTA's shared memory whose bytes are reported to a barrier of the pair's leader
__device__ __forceinline__ void tma_load_2d_pair(void *smem_dst, const void *tmap, int c0, int c1, uint32_t leader_bar)
{
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
                     smem_u32(smem_dst)),
                 "l"(tmap), "r"(leader_bar), "r"(c0), "r"(c1)
                 : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_bar)
{
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
}

// ---------------------------------------------------------------------------------------------------------------
// The same GEMM on CTA pairs (tcgen05 cta_group::2): a cluster of two CTAs owns a 256 x 256 output tile.  Each CTA loads
// its 128 rows of A and its 128 rows (half the columns) of B, so a K block costs a CTA 32 KB instead of 48 KB for the
// same arithmetic (the single-CTA kernel is bound by the L2 -> shared-memory feed), and six stages fit.  The even CTA
// of the pair (the leader) issues the MMAs for both: every 256 x 256 x 32 instruction reads A and B from both CTAs'
// shared memory and accumulates into both CTAs' TMEM (128 rows x 256 columns each).  Both CTAs' TMA loads report to the
// leader's `full` barrier; tcgen05.commit multicasts to both CTAs' `empty` / `acc_full` barriers; both CTAs' epilogue
// warps report to the leader's `acc_empty`.  No TMA load uses cluster multicast.
constexpr int kPairBN = 256;

__global__ void __launch_bounds__(kUmmaThreads, 1) umma2_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                                                                const UmmaArgs a)
{
    constexpr int BN = kPairBN;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    constexpr int kABytes = kUmmaBM * kUmmaBK, kBBytes = (BN / 2) * kUmmaBK, kStageBytes = kABytes + kBBytes; // per CTA
    constexpr int kTmemCols = 2 * BN; // two accumulators: the epilogue drains one while the next tile fills the other
    // 1024-byte alignment as an offset from the array itself: a pointer rebuilt from an integer would lose its address space
    // and every access behind it would compile to a generic load
    uint8_t *smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    float *s_scale = reinterpret_cast<float *>(smem + (size_t)a.stages * kStageBytes); // [2][BN] channel scales of a tile
    int *s_zero = reinterpret_cast<int *>(s_scale + 2 * BN);                            // [2][BN] channel zero points
    uint64_t *bars = reinterpret_cast<uint64_t *>(s_zero + 2 * BN);
    uint64_t *full = bars, *empty = bars + 8, *acc_full = bars + 16, *acc_empty = bars + 18, *par_ready = bars + 20;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 22);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int k_blocks = a.K / kUmmaBK;
    const int m_tiles = (a.M + 2 * kUmmaBM - 1) / (2 * kUmmaBM); // 256-row tiles
    const int total_tiles = m_tiles * ((a.N + BN - 1) / BN);
    const uint32_t rank = cluster_ctarank();                       // 0: leader
    const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;

    if (threadIdx.x == 0) {
        for (int s = 0; s < a.stages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&acc_full[b], 1);
            mbar_init(&acc_empty[b], 8);    // one arrival per epilogue warp of both CTAs (only the leader's is used)
            mbar_init(&par_ready[b], 128);  // every epilogue thread has staged its channel parameters
        }
        fence_mbar_init();
        prefetch_tmap(&tmap_a);
        prefetch_tmap(&tmap_b);
    }
    if (warp == 1) { // TMEM allocation is a warp-wide operation; the same warp frees it at the end
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tmem_fence_before();
    __syncthreads();
    cluster_sync_all(); // the peer's barriers are initialised before anything is signalled across
    tmem_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    pdl_wait_prior_grid(); // operand codes and token sums come from the kernels launched just before

    // Persistent CTA: tiles blockIdx.x, blockIdx.x + gridDim.x, ...; consecutive tiles share the weight (N) tile, so
    // the CTAs running at one time read few distinct weight tiles and all of the activations out of L2.
    if (warp == 0) {
        if (lane == 0) {
            int kc = 0; // k-blocks requested so far, over all tiles
            bool ok = true;
            for (int tile = pair; tile < total_tiles && ok; tile += pairs) {
                const int m0 = (tile % m_tiles) * 2 * kUmmaBM + (int)rank * kUmmaBM, n0 = (tile / m_tiles) * BN + (int)rank * (BN / 2);
                for (int kb = 0; kb < k_blocks; ++kb, ++kc) {
                    const int s = kc % a.stages;
                    if (kc >= a.stages && !mbar_wait_bounded(&empty[s], ((kc / a.stages) - 1) & 1, a.status, STATUS_TIMEOUT_PIPE)) {
                        ok = false;
                        break;
                    }
                    uint8_t *sa = smem + (size_t)s * kStageBytes, *sb = sa + kABytes;
                    if (rank == 0)
                        mbar_arrive_expect_tx(&full[s], 2 * kStageBytes); // both CTAs' bytes land on the leader's barrier
                    const uint32_t leader_full = map_to_cta(smem_u32(&full[s]), 0);
                    tma_load_2d_pair(sa, &tmap_a, kb * kUmmaBK, m0, leader_full);
                    tma_load_2d_pair(sb, &tmap_b, kb * kUmmaBK, n0, leader_full);
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) { // the leader issues for the pair
            int kc = 0, it = 0;
            bool ok = true;
            for (int tile = pair; tile < total_tiles && ok; tile += pairs, ++it) {
                const int b = it & 1;
                if (it >= 2) { // the epilogue has drained this accumulator's previous tile
                    ok = mbar_wait_bounded(&acc_empty[b], ((it >> 1) - 1) & 1, a.status, STATUS_TIMEOUT_PIPE);
                    if (!ok)
                        break;
                    tmem_fence_after();
                }
                const uint32_t tmem_d = tmem_base + (uint32_t)(b * BN);
                for (int kb = 0; kb < k_blocks; ++kb, ++kc) {
                    const int s = kc % a.stages;
                    ok = mbar_wait_bounded(&full[s], (kc / a.stages) & 1, a.status, STATUS_TIMEOUT_TMA);
                    if (!ok)
                        break;
                    tmem_fence_after();
                    const uint32_t sa = smem_u32(smem + (size_t)s * kStageBytes), sb = sa + kABytes;
                    const uint64_t da = make_smem_desc_sw128(sa), db = make_smem_desc_sw128(sb);
#pragma unroll
                    for (int k = 0; k < kUmmaBK / 32; ++k) // 32 bytes of K per instruction: advance the start address inside the atom
                        umma2_i8(tmem_d, da + (uint64_t)(k * 32 >> 4), db + (uint64_t)(k * 32 >> 4), a.idesc, (kb | k) != 0);
                    umma2_commit(&empty[s]); // arrives, in both CTAs, when the MMAs above have finished reading this stage
                }
                if (ok)
                    umma2_commit(&acc_full[b]); // arrives, in both CTAs, when all MMAs of the tile have written the accumulators
            }
        }
        __syncwarp();
    } else {
        // epilogue warps 2..5: a warp may only touch the TMEM lane quarter (warp id % 4)
        const int quarter = warp & 3;
        const int et = threadIdx.x - 64; // 0..127 among the epilogue threads
        const bool channel = a.out_dtype != ABQ_OUT_INT32 && a.scale_mode != ABQ_SCALE_TENSOR_COMPAT;
        const bool has_zero = channel && a.scale_mode == ABQ_SCALE_CHANNEL && a.w_zero != nullptr;
        const __half cscale = a.scale_mode == ABQ_SCALE_TENSOR_COMPAT && a.out_dtype != ABQ_OUT_INT32 ? ld_half(a.C) : __half();
        int it = 0;
        bool ok = true;
        for (int tile = pair; tile < total_tiles && ok; tile += pairs, ++it) {
            const int b = it & 1;
            const int m0 = (tile % m_tiles) * 2 * kUmmaBM + (int)rank * kUmmaBM, n0 = (tile / m_tiles) * BN;
            const int row = m0 + quarter * 32 + lane;
            float *ts = s_scale + b * BN;
            int *tz = s_zero + b * BN;
            if (channel) { // stage the tile's channel parameters while its MMAs still run
                for (int c = et; c < BN; c += 128) {
                    const int n = n0 + c;
                    float sv = 1.f;
                    int zv = 0;
                    if (n < a.N) {
                        if (a.scale_mode == ABQ_SCALE_CHANNEL && a.w_scale)
                            sv = __half2float(a.w_scale[n]);
                        if (has_zero)
                            zv = a.w_zero[n];
                    }
                    ts[c] = sv;
                    tz[c] = zv;
                }
                // epilogue threads only, and bounded like every other wait; the other buffer (tile it - 1) stays untouched
                mbar_arrive(&par_ready[b]);
                ok = mbar_wait_bounded(&par_ready[b], (it >> 1) & 1, a.status, STATUS_TIMEOUT_PIPE);
                if (!ok)
                    break;
            }
            float xs = 1.f;
            int xsum = 0;
            if (row < a.M) {
                if (a.x_scale)
                    xs = a.x_scale[row];
                if (a.xsum)
                    xsum = a.xsum[row];
            }
            ok = mbar_wait_bounded(&acc_full[b], (it >> 1) & 1, a.status, STATUS_TIMEOUT_MMA);
            if (!ok)
                break;
            tmem_fence_after();
#pragma unroll 1
            for (int c = 0; c < BN; c += 32) {
                int v[32];
                tmem_ld32(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(b * BN + c), v);
                if (row >= a.M)
                    continue;
                if (a.out_dtype == ABQ_OUT_INT32)
                    store_chunk<0>(a, v, row, n0 + c, ts + c, tz + c, xs, xsum, cscale, has_zero);
                else if (!channel)
                    store_chunk<1>(a, v, row, n0 + c, ts + c, tz + c, xs, xsum, cscale, has_zero);
                else
                    store_chunk<2>(a, v, row, n0 + c, ts + c, tz + c, xs, xsum, cscale, has_zero);
            }
            tmem_fence_before();
            __syncwarp();
            if (lane == 0)
                mbar_arrive_cluster(map_to_cta(smem_u32(&acc_empty[b]), 0)); // this warp's quarter is free again: tell the leader
        }
    }

    tmem_fence_before();
    __syncthreads();
    cluster_sync_all(); // neither CTA leaves while the other may still signal its barriers or read its shared memory
    if (warp == 1) {
        tmem_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    }
}

// ---------------------------------------------------------------------------------------------------------------
// ABQ_SCALE_GROUP on the tensor-core route: every scale group (kb_per_group K blocks) is multiplied into a fresh TMEM
// accumulator, exactly, and the epilogue warps drain it while the next group is multiplied into the other one:
//     facc[n] += scale[n][g] * acc_g[n]                                              (fp32, one row per thread)
// The zero points are not seen here: the weight codes in the scratch are w - zero[n][g] (signed int8, exact for widths
// up to 7 bits; see unpack_i8), so acc_g already is sum x * (w - z).  BN = 128 columns (128 fp32 partial sums per
// thread); the scales of the tile, all groups, are staged once per tile in shared memory as fp32 [group][column].
// MAGIC: |acc_g| < 2^22 (signed 8-bit activations, one K block per group): int -> float by the 1.5 * 2^23 trick, two
// pipelined operations instead of a conversion instruction.  Same roles, barriers and bounded waits as umma_kernel.
// facc[C .. C + 31] += scale[C .. C + 31] * float(v[0 .. 31]); the scales are the same for every lane (shared-memory broadcast)
template <bool MAGIC, int C>
__device__ __forceinline__ void scale_add(const int (&v)[32], const float *scales, float (&facc)[64])
{
#pragma unroll
    for (int j = 0; j < 32; j += 4) {
        const float4 sc = *reinterpret_cast<const float4 *>(scales + C + j);
        const float s4[4] = { sc.x, sc.y, sc.z, sc.w };
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float fv = MAGIC ? __int_as_float(v[j + e] + 0x4b400000) - 12582912.0f : (float)v[j + e];
            facc[C + j + e] = fmaf(s4[e], fv, facc[C + j + e]);
        }
    }
}

constexpr int kGroupBN = 128;
constexpr int kGroupThreads = 320; // TMA warp, MMA warp, eight epilogue warps: two per TMEM lane quarter, 64 columns each

template <bool MAGIC>
__global__ void __launch_bounds__(kGroupThreads, 1) umma_group_kernel(const __grid_constant__ CUtensorMap tmap_a,
                                                                     const __grid_constant__ CUtensorMap tmap_b, const UmmaArgs a)
{
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    constexpr int BN = kGroupBN;
    constexpr int kABytes = kUmmaBM * kUmmaBK, kBBytes = BN * kUmmaBK, kStageBytes = kABytes + kBBytes;
    constexpr int kAccs = 4;              // accumulators in flight: the hand-over MMA -> epilogue -> MMA takes longer than two groups
    constexpr int kTmemCols = kAccs * BN; // all 512 columns
    // 1024-byte alignment as an offset from the array itself: a pointer rebuilt from an integer would lose its address space
    // and every access behind it would compile to a generic load
    uint8_t *smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    const int G = a.scale_groups;
    float *s_scale = reinterpret_cast<float *>(smem + (size_t)a.stages * kStageBytes); // [G][BN]
    uint64_t *bars = reinterpret_cast<uint64_t *>(s_scale + (size_t)G * BN);
    uint64_t *full = bars, *empty = bars + 8, *acc_full = bars + 16, *acc_empty = bars + 20, *par_ready = bars + 24, *par_free = bars + 25;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 26);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int k_blocks = a.K / kUmmaBK;
    const int m_tiles = (a.M + kUmmaBM - 1) / kUmmaBM;
    const int total_tiles = m_tiles * ((a.N + BN - 1) / BN);

    if (threadIdx.x == 0) {
        for (int s = 0; s < a.stages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int b = 0; b < kAccs; ++b) {
            mbar_init(&acc_full[b], 1);
            mbar_init(&acc_empty[b], 8);
        }
        mbar_init(par_ready, 256); // the tile's scales are staged
        mbar_init(par_free, 256);  // ... and no longer read (the next tile may overwrite them)
        fence_mbar_init();
        prefetch_tmap(&tmap_a);
        prefetch_tmap(&tmap_b);
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tmem_fence_before();
    __syncthreads();
    tmem_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    pdl_wait_prior_grid();

    if (warp == 0) {
        if (lane == 0) {
            int kc = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
                const int m0 = (tile % m_tiles) * kUmmaBM, n0 = (tile / m_tiles) * BN;
                for (int kb = 0; kb < k_blocks; ++kb, ++kc) {
                    const int s = kc % a.stages;
                    if (kc >= a.stages && !mbar_wait_bounded(&empty[s], ((kc / a.stages) - 1) & 1, a.status, STATUS_TIMEOUT_PIPE)) {
                        ok = false;
                        break;
                    }
                    uint8_t *sa = smem + (size_t)s * kStageBytes, *sb = sa + kABytes;
                    mbar_arrive_expect_tx(&full[s], kStageBytes);
                    tma_load_2d(sa, &tmap_a, kb * kUmmaBK, m0, &full[s]);
                    tma_load_2d(sb, &tmap_b, kb * kUmmaBK, n0, &full[s]);
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        if (lane == 0) {
            int kc = 0, gc = 0; // K blocks and scale groups issued so far, over all tiles
            bool ok = true;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
                if (a.kb_per_group == 0) {
                    // scale groups of 64 features: a K block holds two groups; its first two MMAs start one accumulator, its
                    // last two the next
                    for (int kb = 0; kb < k_blocks && ok; ++kb, ++kc) {
                        const int s = kc % a.stages;
                        ok = mbar_wait_bounded(&full[s], (kc / a.stages) & 1, a.status, STATUS_TIMEOUT_TMA);
                        if (!ok)
                            break;
                        tmem_fence_after();
                        const uint32_t sa = smem_u32(smem + (size_t)s * kStageBytes), sb = sa + kABytes;
                        const uint64_t da = make_smem_desc_sw128(sa), db = make_smem_desc_sw128(sb);
                        for (int h = 0; h < 2 && ok; ++h, ++gc) {
                            const int b = gc % kAccs;
                            if (gc >= kAccs) {
                                ok = mbar_wait_bounded(&acc_empty[b], ((gc / kAccs) - 1) & 1, a.status, STATUS_TIMEOUT_PIPE);
                                if (!ok)
                                    break;
                                tmem_fence_after();
                            }
                            const uint32_t tmem_d = tmem_base + (uint32_t)(b * BN);
#pragma unroll
                            for (int k = 0; k < 2; ++k)
                                umma_i8(tmem_d, da + (uint64_t)((2 * h + k) * 32 >> 4), db + (uint64_t)((2 * h + k) * 32 >> 4), a.idesc, k != 0);
                            umma_commit(&acc_full[b]);
                        }
                        if (ok)
                            umma_commit(&empty[s]);
                    }
                    continue;
                }
                for (int g = 0; g < G && ok; ++g, ++gc) {
                    const int b = gc % kAccs;
                    if (gc >= kAccs) { // the epilogue has drained this accumulator's previous group
                        ok = mbar_wait_bounded(&acc_empty[b], ((gc / kAccs) - 1) & 1, a.status, STATUS_TIMEOUT_PIPE);
                        if (!ok)
                            break;
                        tmem_fence_after();
                    }
                    const uint32_t tmem_d = tmem_base + (uint32_t)(b * BN);
                    for (int kg = 0; kg < a.kb_per_group; ++kg, ++kc) {
                        const int s = kc % a.stages;
                        ok = mbar_wait_bounded(&full[s], (kc / a.stages) & 1, a.status, STATUS_TIMEOUT_TMA);
                        if (!ok)
                            break;
                        tmem_fence_after();
                        const uint32_t sa = smem_u32(smem + (size_t)s * kStageBytes), sb = sa + kABytes;
                        const uint64_t da = make_smem_desc_sw128(sa), db = make_smem_desc_sw128(sb);
#pragma unroll
                        for (int k = 0; k < kUmmaBK / 32; ++k) // the first MMA of a group starts a fresh sum
                            umma_i8(tmem_d, da + (uint64_t)(k * 32 >> 4), db + (uint64_t)(k * 32 >> 4), a.idesc, (kg | k) != 0);
                        umma_commit(&empty[s]);
                    }
                    if (ok)
                        umma_commit(&acc_full[b]);
                }
            }
        }
        __syncwarp();
    } else {
        const int quarter = warp & 3;          // the TMEM lanes a warp may read: 32 * (warp id % 4)
        const int half = (warp - 2) >> 2;      // which 64 of the tile's 128 columns
        const int et = threadIdx.x - 64;       // 0..255
        constexpr int HN = BN / 2;
        int gc = 0, it = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++it) {
            const int m0 = (tile % m_tiles) * kUmmaBM, n0 = (tile / m_tiles) * BN;
            const int row = m0 + quarter * 32 + lane;
            // ---- stage the scales of weight row n0 + et, all groups, as [group][column]
            if (it > 0) {
                ok = mbar_wait_bounded(par_free, (it - 1) & 1, a.status, STATUS_TIMEOUT_PIPE);
                if (!ok)
                    break;
            }
            {
                const int col = et & (BN - 1), n = n0 + col;
                const __half *src = a.w_scale + (size_t)(n < a.N ? n : 0) * G;
                for (int g = et >> 7; g < G; g += 2) // two threads per weight row, alternate groups
                    s_scale[(size_t)g * BN + col] = n < a.N ? __half2float(src[g]) : 0.f;
            }
            mbar_arrive(par_ready);
            ok = mbar_wait_bounded(par_ready, it & 1, a.status, STATUS_TIMEOUT_PIPE);
            if (!ok)
                break;
            float xs = 1.f;
            if (row < a.M && a.x_scale)
                xs = a.x_scale[row];
            float facc[HN];
#pragma unroll
            for (int c = 0; c < HN; ++c)
                facc[c] = 0.f;
            // Pipelined over 32-column chunks: while chunk i is scaled and added, the tcgen05.ld of chunk i + 1 (the second
            // half of this group, or the first half of the next group) is already in flight; an accumulator goes back
            // to the MMA warp as soon as its second half sits in registers.
            int va[32], vb[32];
            const uint32_t tlane = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(half * HN);
            {
                const int b = gc % kAccs;
                ok = mbar_wait_bounded(&acc_full[b], (gc / kAccs) & 1, a.status, STATUS_TIMEOUT_MMA);
                if (!ok)
                    break;
                tmem_fence_after();
                tmem_ld32_nowait(tlane + (uint32_t)(b * BN), va);
            }
            for (int g = 0; g < G; ++g) {
                const int b = gc % kAccs;
                const float *sg = s_scale + (size_t)g * BN + half * HN;
                tmem_ld_wait();                                         // first half of group g is in va
                tmem_ld32_nowait(tlane + (uint32_t)(b * BN + 32), vb);  // second half on its way
                scale_add<MAGIC, 0>(va, sg, facc);
                tmem_ld_wait();                                         // second half in vb: the accumulator is free
                tmem_fence_before();
                __syncwarp();
                if (lane == 0)
                    mbar_arrive(&acc_empty[b]);
                ++gc;
                if (g + 1 < G) {
                    const int nb = gc % kAccs;
                    ok = mbar_wait_bounded(&acc_full[nb], (gc / kAccs) & 1, a.status, STATUS_TIMEOUT_MMA);
                    if (!ok)
                        break;
                    tmem_fence_after();
                    tmem_ld32_nowait(tlane + (uint32_t)(nb * BN), va);  // first half of group g + 1 on its way
                }
                scale_add<MAGIC, 32>(vb, sg, facc);
            }
            mbar_arrive(par_free); // this thread reads the staged parameters no more
            if (!ok)
                break;
            if (row < a.M) {
                const int nb = n0 + half * HN;
                __half *dst = reinterpret_cast<__half *>(a.D) + (size_t)row * a.N + nb;
                const bool vec = nb + HN <= a.N && (a.N & 7) == 0;
#pragma unroll
                for (int c = 0; c < HN; c += 8) {
                    uint32_t h[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const __half2 t = __floats2half2_rn(facc[c + 2 * e] * xs, facc[c + 2 * e + 1] * xs);
                        h[e] = *reinterpret_cast<const uint32_t *>(&t);
                    }
                    if (vec) {
                        *reinterpret_cast<uint4 *>(dst + c) = make_uint4(h[0], h[1], h[2], h[3]);
                    } else {
#pragma unroll
                        for (int e = 0; e < 8; ++e)
                            if (nb + c + e < a.N)
                                dst[c + e] = __ushort_as_half((unsigned short)(h[e >> 1] >> ((e & 1) * 16)));
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
    const uint4 *p = reinterpret_cast<const uint4 *>(x + (size_t)row * K); // K is a multiple of 128: rows are 16-byte aligned
    int s = 0;
    const int n16 = K / 16;
#pragma unroll 8
    for (int i = lane; i < n16; i += 32) {
        const uint4 w = __ldg(p + i);
        if (is_signed) {
            s = __dp4a((int)w.x, 0x01010101, s);
            s = __dp4a((int)w.y, 0x01010101, s);
            s = __dp4a((int)w.z, 0x01010101, s);
            s = __dp4a((int)w.w, 0x01010101, s);
        } else {
            unsigned u = (unsigned)s;
            u = __dp4a(w.x, 0x01010101u, u);
            u = __dp4a(w.y, 0x01010101u, u);
            u = __dp4a(w.z, 0x01010101u, u);
            u = __dp4a(w.w, 0x01010101u, u);
            s = (int)u;
        }
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
    const bool grouped = p.scale_mode == ABQ_SCALE_GROUP;
    const int scale_groups = grouped ? p.K / p.group_size : 0;
    if (grouped) {
        // drained per scale group (umma_group_kernel): groups of whole K blocks; zero points are folded into the int8
        // weight codes, which needs w - z to fit: unsigned weights of at most 7 bits
        if ((p.group_size % kUmmaBK != 0 && p.group_size != kUmmaBK / 2) || p.out_dtype != ABQ_OUT_FP16)
            return ABQ_ERR_UNSUPPORTED; // (groups of 64: two per K block, see the MMA warp of umma_group_kernel)
        if (p.w_zero && (p.w_signed || p.w_bits > 7))
            return ABQ_ERR_UNSUPPORTED;
        if ((size_t)scale_groups * kGroupBN * 4 + 3 * (size_t)(kUmmaBM + kGroupBN) * kUmmaBK > 216 * 1024)
            return ABQ_ERR_UNSUPPORTED; // the tile's scales would not fit beside three stages
    }
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
    // N tile: the persistent CTAs run ceil(tiles / SMs) tiles each.  Narrower tiles balance better, but measured per
    // output column they cost almost twice as much (operand fetch per operation doubles), so they only win on small grids
    const int m_tiles = (p.M + kUmmaBM - 1) / kUmmaBM;
    int BN = 256;
    {
        double best = 0;
        for (int bn = 256; bn >= 64; bn >>= 1) {
            const long tiles = (long)m_tiles * ((p.N + bn - 1) / bn);
            const double t = (double)((tiles + sms - 1) / sms) * bn * (bn == 256 ? 1.0 : (bn == 128 ? 1.85 : 3.5));
            if (best == 0 || t < best) {
                best = t;
                BN = bn;
            }
        }
    }
    BN = env_int("ABQ_UMMA_BN", BN);
    if (BN != 64 && BN != 128 && BN != 256)
        return ABQ_ERR_INVALID_ARG;
    if (grouped)
        BN = kGroupBN;
    // CTA pairs (256 x 256 tiles, umma2_kernel): a third less operand traffic per SM and six stages.  Measured equal to the
    // single-CTA kernel on the LLaMA shapes (that one already runs at the rate its rounds of tiles allow), so it is
    // opt-in: ABQ_UMMA_PAIRS=1
    const bool paired = !grouped && BN == 256 && p.M > kUmmaBM && env_int("ABQ_UMMA_PAIRS", 0) != 0;
    const int stage_bytes = paired ? (kUmmaBM + kPairBN / 2) * kUmmaBK : (kUmmaBM + BN) * kUmmaBK;
    const size_t param_bytes = grouped ? (size_t)scale_groups * kGroupBN * 4 : (size_t)4 * BN * 4;
    int stages = (int)((216 * 1024 - param_bytes) / stage_bytes);
    stages = stages > 8 ? 8 : stages;
    const int k_blocks = p.K / kUmmaBK;
    stages = stages > k_blocks ? k_blocks : stages;
    stages = env_int("ABQ_UMMA_STAGES", stages);
    if (stages < 1 || stages > 8)
        return ABQ_ERR_INVALID_ARG;

    uint8_t *ws = reinterpret_cast<uint8_t *>(p.workspace);
    const uint64_t dims_a[2] = { (uint64_t)p.K, (uint64_t)p.M }, dims_b[2] = { (uint64_t)p.K, (uint64_t)p.N };
    const uint64_t strides[1] = { (uint64_t)p.K };
    const uint32_t box_a[2] = { (uint32_t)kUmmaBK, (uint32_t)kUmmaBM }, box_b[2] = { (uint32_t)kUmmaBK, (uint32_t)(paired ? kPairBN / 2 : BN) };
    if (!encode_tmap(st->tmap[0], TMAP_U8, 2, ws, dims_a, strides, box_a, TMAP_SWIZZLE_128B) ||
        !encode_tmap(st->tmap[1], TMAP_U8, 2, ws + off_w, dims_b, strides, box_b, TMAP_SWIZZLE_128B))
        return ABQ_ERR_CUDA;
    long tiles = (long)m_tiles * ((p.N + BN - 1) / BN);
    if (paired) { // 256-row tiles, two CTAs each
        tiles = (long)((p.M + 2 * kUmmaBM - 1) / (2 * kUmmaBM)) * ((p.N + kPairBN - 1) / kPairBN);
        const long pairs = tiles < sms / 2 ? tiles : sms / 2;
        st->grid[0] = (unsigned)(2 * pairs);
    } else
        st->grid[0] = (unsigned)(tiles < sms ? tiles : sms); // persistent: a CTA per SM, tiles dealt round-robin
    st->grid[1] = 1;
    st->grid[2] = 1;
    st->block[0] = grouped ? kGroupThreads : kUmmaThreads;
    st->block[1] = st->block[2] = 1;
    st->cluster = paired ? 2 : 1;
    st->shared_mem_size = 1024 + (size_t)stages * stage_bytes + param_bytes + 256;
    st->tile[0] = BN;
    st->tile[1] = stages;
    st->tile[2] = grouped ? 1 : (paired ? 2 : 0);
    return ABQ_OK;
}

template <typename Kernel>
static cudaError_t launch_kernel(Kernel kern, SmemOptIn *opted, const abq_gemm_state *st, const UmmaArgs &args, cudaStream_t stream)
{
    const int threads = st->block[0];
    {
        cudaError_t e = opted->ensure(kern, st->shared_mem_size);
        if (e != cudaSuccess)
            return e;
    }
    CUtensorMap ta, tb;
    memcpy(&ta, st->tmap[0], sizeof(ta));
    memcpy(&tb, st->tmap[1], sizeof(tb));
    // programmatic launch: barrier set-up, TMEM allocation and descriptor prefetch overlap the tail of the expansion
    // kernel; every thread passes griddepcontrol.wait before it touches what that kernel (or the token sums) wrote
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(st->grid[0], 1, 1);
    cfg.blockDim = dim3(threads);
    cfg.dynamicSmemBytes = st->shared_mem_size;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (st->cluster == 2) {
        attr[1].id = cudaLaunchAttributeClusterDimension;
        attr[1].val.clusterDim.x = 2;
        attr[1].val.clusterDim.y = 1;
        attr[1].val.clusterDim.z = 1;
        cfg.numAttrs = 2;
    }
    return cudaLaunchKernelEx(&cfg, kern, ta, tb, args);
}

template <bool MAGIC>
static cudaError_t launch_group(const abq_gemm_state *st, const UmmaArgs &args, cudaStream_t stream)
{
    static thread_local SmemOptIn opted;
    return launch_kernel(umma_group_kernel<MAGIC>, &opted, st, args, stream);
}

static cudaError_t launch_pair(const abq_gemm_state *st, const UmmaArgs &args, cudaStream_t stream)
{
    static thread_local SmemOptIn opted;
    return launch_kernel(umma2_kernel, &opted, st, args, stream);
}

template <int BN>
static cudaError_t launch_bn(const abq_gemm_state *st, const UmmaArgs &args, cudaStream_t stream)
{
    static thread_local SmemOptIn opted;
    return launch_kernel(umma_kernel<BN>, &opted, st, args, stream);
}

// Zero points that the weight expansion subtracts (the codes multiplied are then w - zero, signed): always with per-group
// scales on this route (the plan has checked that the difference fits int8), with per-channel scales where it fits
// (unsigned weights of at most 7 bits); otherwise the epilogue subtracts zero * sum(x).
static const uint8_t *folded_zero(const abq_gemm_params &p)
{
    if (p.scale_mode == ABQ_SCALE_GROUP)
        return p.w_zero;
    if (p.scale_mode == ABQ_SCALE_CHANNEL && p.out_dtype == ABQ_OUT_FP16 && !p.w_signed && p.w_bits <= 7)
        return p.w_zero;
    return nullptr;
}
static int folded_group(const abq_gemm_params &p) { return p.scale_mode == ABQ_SCALE_GROUP ? p.group_size : p.K; }

cudaError_t umma_prepare_weights(const abq_gemm_state *st, cudaStream_t stream)
{
    const abq_gemm_params &p = st->p;
    size_t off_w, off_sum, total;
    umma_layout(p.M, p.N, p.K, &off_w, &off_sum, &total);
    return unpack_i8(reinterpret_cast<const uint32_t *>(p.W), reinterpret_cast<uint8_t *>(p.workspace) + off_w, p.N, p.K, p.w_bits, p.w_signed,
                     stream, folded_zero(p), folded_group(p));
}

cudaError_t umma_launch(const abq_gemm_state *st, cudaStream_t stream)
{
    const abq_gemm_params &p = st->p;
    size_t off_w, off_sum, total;
    umma_layout(p.M, p.N, p.K, &off_w, &off_sum, &total);
    uint8_t *ws = reinterpret_cast<uint8_t *>(p.workspace);
    cudaError_t e;
    if (p.flags & ABQ_FLAG_X_HALF) { // fp16 activations: quantise straight to codes; weights as usual
        e = cudaSuccess;
        if (!(p.flags & ABQ_FLAG_WEIGHTS_PREPARED))
            e = unpack_i8(reinterpret_cast<const uint32_t *>(p.W), ws + off_w, p.N, p.K, p.w_bits, p.w_signed, stream, folded_zero(p),
                          folded_group(p));
        if (e == cudaSuccess)
            e = quantize_codes(p.X, p.x_quant_scale, ws, p.M, p.K, p.x_bits, stream);
    } else if (p.flags & ABQ_FLAG_WEIGHTS_PREPARED) // the weight codes are in place: expand the activations only
        e = unpack_i8(reinterpret_cast<const uint32_t *>(p.X), ws, p.M, p.K, p.x_bits, p.x_signed, stream);
    else
        e = unpack_pair_i8(reinterpret_cast<const uint32_t *>(p.X), ws, p.M, p.x_bits, p.x_signed, reinterpret_cast<const uint32_t *>(p.W),
                           ws + off_w, p.N, p.w_bits, p.w_signed, p.K, stream, folded_zero(p), folded_group(p));
    if (e != cudaSuccess)
        return e;
    UmmaArgs a;
    a.xsum = nullptr;
    if (p.scale_mode == ABQ_SCALE_CHANNEL && p.w_zero && !folded_zero(p)) {
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
    a.w_zero = folded_zero(p) ? nullptr : p.w_zero;
    a.x_scale = p.x_scale;
    a.out_dtype = p.out_dtype;
    a.scale_mode = p.scale_mode;
    const int BN = st->tile[0];
    // instruction descriptor, kind::i8: D format S32 (2) at bit 4, A / B format (0 = U8, 1 = S8) at bits 7 / 10,
    // both operands K-major (bits 15, 16 clear), N >> 3 at bit 17, M >> 4 at bit 24
    const bool b_signed = p.w_signed || folded_zero(p) != nullptr; // w - zero is a signed code
    a.idesc = (2u << 4) | ((p.x_signed ? 1u : 0u) << 7) | ((b_signed ? 1u : 0u) << 10) | ((uint32_t)(BN >> 3) << 17) |
              ((uint32_t)(kUmmaBM >> 4) << 24);
    a.status = p.status_word;
    a.kb_per_group = p.scale_mode == ABQ_SCALE_GROUP ? p.group_size / kUmmaBK : 0;
    a.scale_groups = p.scale_mode == ABQ_SCALE_GROUP ? p.K / p.group_size : 0;
    if (st->tile[2] == 2) { // CTA pairs: one instruction covers 256 rows
        a.idesc = (a.idesc & ~(0x1fu << 24)) | ((uint32_t)(2 * kUmmaBM >> 4) << 24);
        return launch_pair(st, a, stream);
    }
    if (st->tile[2]) {
        // |acc of a group| < 2^22 with signed activations (|x| <= 128), |w - z| <= 255 and one K block per group
        const bool magic = p.x_signed && a.kb_per_group <= 1;
        return magic ? launch_group<true>(st, a, stream) : launch_group<false>(st, a, stream);
    }
    switch (BN) {
    case 64: return launch_bn<64>(st, a, stream);
    case 128: return launch_bn<128>(st, a, stream);
    default: return launch_bn<256>(st, a, stream);
    }
}

} // namespace abq
