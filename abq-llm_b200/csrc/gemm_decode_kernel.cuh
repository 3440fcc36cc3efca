// Decode-shape GEMM (up to 16 rows per launch), route ABQ_ROUTE_I8_MMA: one kernel per GEMM.
//
// HBM-bound and, at LLaMA sizes, only a few microseconds long, so the kernel is built around two things:
// every weight plane word is read exactly once, and nothing on the path from "activations are ready" to "output
// is written" goes through global memory more often than it must.
//
//  * One CTA of 16 warps per SM.  CTA c owns an even share of the 16-row weight tiles.  `split` warps share a
//    tile, each taking a contiguous range of 512-feature stages, so that all 16 warps have work even when a CTA
//    has only one or two tiles; their partial sums meet in shared memory (mbarrier hand-shake, fixed order).
//  * Every warp feeds itself: lane 0 issues 3-D TMA boxes (all q planes x 16 rows x 512 input features, 64-byte
//    rows, 64B-swizzled) into a warp-private ring and refills a slot right after the warp has consumed it, across
//    tile boundaries.  Weight requests go out before the dependency wait of a programmatic dependent launch:
//    weights never depend on the previous kernel.
//  * The activations arrive as bit-planes; after the dependency wait the CTA expands the planes of its K range
//    once into "records" in shared memory: the B fragments of mma.sync.m16n8k32 in the order the warps read them,
//    plus per-128-feature code sums (for zero points and offset-coded signed weights).
//  * A thread takes one 32-bit word per plane and row and recombines the q plane words into byte codes with a
//    butterfly (expand.cuh); the bytes are the A operand of the MMA (u8 x s8/u8 -> s32).  Two accumulator sets
//    carry different power-of-two scales, which saves the shifts that would otherwise normalise the bit fields.
//  * Scale / zero-point dequantisation is fused: per scale group the int32 accumulators are folded into fp32.
//  * Only when the records of the whole K range do not fit in shared memory is K also split over CTAs; those
//    partials go through a workspace slot per slice and the CTA arriving last at the tile's counter adds them in
//    slice order.
//
// Covers what the reference does with plane-stacked 1-bit MMAs and an smem shift-accumulate epilogue
// (engine/mma_any/aq_bmma_kernel.h:109-271, 485-580), with its fp16 scalar-scale epilogue
// (fastertransformer/.../abqgemm/mma_any/aq_bmma_kernel.h:474-524), and with the activation side of the plane
// stacking (aq_bmma_kernel.h:146-152).
//
// This header holds the kernel and its launch templates; gemm_decode_w1.cu .. gemm_decode_w8.cu instantiate them for one
// weight width each (so that the widths compile in parallel), gemm_decode.cu holds the planner and the launch entry.
#pragma once
#include <cuda.h>
#include <cstring>

#include "abq_common.cuh"
#include "abq_kernels.h"
#include "expand.cuh"
#include "xbytes.cuh"

namespace abq {

constexpr int kMaxRing = 6;
constexpr int kMaxWarps = 16;

struct DecodeArgs {
    int M, N, K;
    int tiles;             // ceil(N / 16)
    int total_groups;      // K / 128
    int slices;            // K split over CTAs (1 unless the records of all K do not fit in shared memory)
    int stages_per_slice;  // 512-feature stages per slice
    int ctas_per_slice;
    int split;             // warps sharing one tile
    int stages_per_split;  // stages per warp of a tile
    int ring;              // TMA stages per warp
    const uint32_t *X;     // activation planes [x_bits][rows][K/32], first row of this launch
    size_t x_plane_words;  // words between two planes (all rows of the operand, not only the M of this launch)
    const float *x_qscale; // not null: X is fp16 [rows][K], quantised here with this static scale (see build_records_half)
    int x_bits, x_signed;
    int *counters;         // one per tile (slices > 1), zero before the launch, left zero after it
    int *partials;         // [slice][tile][token][16 rows] int32 or fp32 bit patterns (slices > 1)
    void *D;
    const __half *w_scale;
    const uint8_t *w_zero;
    const float *x_scale;
    const __half *C;
    int out_dtype, scale_mode;
    int groups_per_scale; // 128-feature groups per scale group (GROUP mode)
    int scale_groups;     // scale groups per weight row
    int w_signed;
    int *status;
    const __half *residual; // not null: added (fp16) to the fp16 result before it is stored
    // worked out once on the host instead of by every thread of every launch (each an integer division there):
    int tiles_q, tiles_r;    // tiles / ctas_per_slice and the remainder: the first tiles_r CTAs of a slice take one tile more
    int tiles_per_round;     // warps of the CTA / split
    uint32_t split_magic;    // warp / split == umulhi(warp, split_magic)
    uint32_t words_magic;    // idx / (4 * stages_per_slice * 4) == umulhi(idx, words_magic): record items of a full slice
};

// Expand the activation planes of groups [g_first, g_first + n_groups) into records in shared memory.  Record of a
// 128-feature group: [token tile mt][step pair ip][lane = 4 g + t][16 bytes] B fragments, then 16 int32 code sums.
// The 16 bytes of (mt, ip, lane) are registers r[4 ip .. 4 ip + 3] of token 8 mt + g and 32-feature run t.
template <int P, int NW>
__device__ __forceinline__ void build_records(const DecodeArgs &a, uint8_t *rec_base, int g_first, int n_groups, int MT, int rec_bytes)
{
    const int KW = a.K >> 5;
    const int words = n_groups * 4;
    const int items = MT * 8 * words;
    const size_t plane = a.x_plane_words;
    // idx / words by a multiplication (a few thousand items at most); the host knows the divisor of a slice with all its stages
    const uint32_t magic = words == a.stages_per_slice * 16 ? a.words_magic : 0xffffffffu / (uint32_t)max(words, 1) + 1u;
    for (int idx = threadIdx.x; idx < items; idx += NW * 32) {
        const int m = (int)__umulhi((uint32_t)idx, magic), kwl = idx - m * words;
        uint32_t r[8];
        int sum = 0;
        if (m < a.M) {
            uint32_t p[P];
            const uint32_t *src = a.X + (size_t)m * KW + g_first * 4 + kwl;
#pragma unroll
            for (int b = 0; b < P; ++b)
                p[b] = __ldg(src + b * plane);
            x_bytes<P>(p, a.x_signed != 0, r);
            if (a.x_signed) {
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
        } else {
#pragma unroll
            for (int s = 0; s < 8; ++s)
                r[s] = 0;
        }
        // the four 32-feature runs of a group sit in four consecutive lanes (words is a multiple of 4)
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        const int G = kwl >> 2, t = kwl & 3, mt = m >> 3, g = m & 7;
        uint8_t *rec = rec_base + (size_t)G * rec_bytes;
        uint4 *dst = reinterpret_cast<uint4 *>(rec + ((mt * 2) * 32 + g * 4 + t) * 16);
        dst[0] = make_uint4(r[0], r[1], r[2], r[3]);
        dst[32] = make_uint4(r[4], r[5], r[6], r[7]);
        if (t == 0)
            reinterpret_cast<int *>(rec + 1024 * MT)[m] = sum;
    }
}

// The same records straight from fp16 activations: code = (int)(half(x) * half(scale)), truncated, the low x_bits bits
// kept and sign-extended -- what quantize_pack_half (mode 0) followed by build_records gives, without the planes.
template <int NW>
__device__ __forceinline__ void build_records_half(const DecodeArgs &a, uint8_t *rec_base, int g_first, int n_groups, int MT, int rec_bytes)
{
    const int words = n_groups * 4;
    const int items = MT * 8 * words;
    const __half *xh = reinterpret_cast<const __half *>(a.X);
    const __half hscale = __float2half(__ldg(a.x_qscale));
    const uint32_t keep = 0x01010101u * ((1u << a.x_bits) - 1u);
    const uint32_t magic = words == a.stages_per_slice * 16 ? a.words_magic : 0xffffffffu / (uint32_t)max(words, 1) + 1u;
    for (int idx = threadIdx.x; idx < items; idx += NW * 32) {
        const int m = (int)__umulhi((uint32_t)idx, magic), kwl = idx - m * words;
        uint32_t r[8];
#pragma unroll
        for (int s = 0; s < 8; ++s)
            r[s] = 0;
        int sum = 0;
        if (m < a.M) {
            const uint4 *src = reinterpret_cast<const uint4 *>(xh + (size_t)m * a.K + (size_t)(g_first * 4 + kwl) * 32);
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
#pragma unroll
            for (int s = 0; s < 8; ++s) {
                r[s] &= keep;
                if (a.x_bits < 8)
                    r[s] = sign_extend_bytes(r[s], a.x_bits);
                sum = __dp4a((int)r[s], 0x01010101, sum);
            }
        }
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        const int G = kwl >> 2, t = kwl & 3, mt = m >> 3, g = m & 7;
        uint8_t *rec = rec_base + (size_t)G * rec_bytes;
        uint4 *dst = reinterpret_cast<uint4 *>(rec + ((mt * 2) * 32 + g * 4 + t) * 16);
        dst[0] = make_uint4(r[0], r[1], r[2], r[3]);
        dst[32] = make_uint4(r[4], r[5], r[6], r[7]);
        if (t == 0)
            reinterpret_cast<int *>(rec + 1024 * MT)[m] = sum;
    }
}

template <int Q, int MT, bool XU8, bool GROUPED, bool GPS1, int NW>
__global__ void __launch_bounds__(NW * 32, 1) decode_kernel(const __grid_constant__ CUtensorMap tmap_w, const DecodeArgs a)
{
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    constexpr int kStageBytes = Q * 1024; // [plane][16 rows][64 B]
    constexpr int kRec = decode_record_bytes(MT);
    using X = Expand<Q>;
    // 1024-byte alignment as an offset from the array itself: a pointer rebuilt from an integer would lose its address space
    // and every access behind it would compile to a generic load
    uint8_t *smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    uint8_t *ring_base = smem;
    uint8_t *rec_base = ring_base + (size_t)NW * a.ring * kStageBytes;
    int *red = reinterpret_cast<int *>(rec_base + (size_t)a.stages_per_slice * 4 * kRec); // [warp][4 MT][32 lanes]
    uint64_t *bars = reinterpret_cast<uint64_t *>(red + NW * 4 * MT * 32);
    uint64_t *full = bars;                      // [warp][slot]: TMA stage landed
    uint64_t *red_ready = bars + NW * kMaxRing; // [tile slot]: partials of the other warps of the tile are written
    uint64_t *red_free = red_ready + NW;        // [tile slot]: the reducing warp has read them

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int s = a.slices > 1 ? blockIdx.x / a.ctas_per_slice : 0; // K-slice of this CTA
    const int cb = blockIdx.x - s * a.ctas_per_slice;               // position among the CTAs of the slice
    // tiles [r_begin, r_end): an even share, the first tiles_r CTAs of the slice taking one more
    const int r_begin = cb * a.tiles_q + min(cb, a.tiles_r);
    const int r_end = r_begin + a.tiles_q + (cb < a.tiles_r ? 1 : 0);
    const int total_stages = (a.total_groups + 3) >> 2;
    const int slice_first = s * a.stages_per_slice;                                     // first stage of the slice
    const int slice_nst = max(0, min(total_stages - slice_first, a.stages_per_slice)); // its stage count
    const int g_slice = slice_first * 4;                                                // its first 128-group
    const int n_groups = max(0, min(a.total_groups - g_slice, a.stages_per_slice * 4));

    // role of this warp: tile slot ts of the round, part sc of that tile's stages
    const int tiles_per_round = a.tiles_per_round;
    const int ts = a.split == 1 ? warp : (int)__umulhi((uint32_t)warp, a.split_magic), sc = warp - ts * a.split; // (no magic for 1)
    const bool active = ts < tiles_per_round;
    const int st_begin = min(slice_nst, sc * a.stages_per_split); // stages [st_begin, st_end) of the slice
    const int st_end = min(slice_nst, st_begin + a.stages_per_split);
    const int my_nst = active ? st_end - st_begin : 0;

    if (lane == 0) { // every warp sets up its own barriers
        for (int i = 0; i < a.ring; ++i)
            mbar_init(&full[warp * kMaxRing + i], 1);
        mbar_init(&red_ready[warp], a.split > 1 ? a.split - 1 : 1);
        mbar_init(&red_free[warp], 1);
        fence_mbar_init();
    }
    __syncthreads();
    pdl_launch_dependents();

    // ---- request side (lane 0 of every warp): cursor over (tile, stage) in the order the warp consumes them
    int ir = r_begin + ts, ij = 0;
    uint8_t *my_ring = ring_base + (size_t)warp * a.ring * kStageBytes;
    uint64_t *my_full = full + warp * kMaxRing;
    auto issue = [&](int slot) {
        mbar_arrive_expect_tx(&my_full[slot], kStageBytes);
        tma_load_3d(my_ring + (size_t)slot * kStageBytes, &tmap_w, (slice_first + st_begin + ij) * 16, ir * 16, 0, &my_full[slot]);
        if (++ij == my_nst) {
            ij = 0;
            ir += tiles_per_round;
        }
    };
    if (lane == 0 && my_nst > 0) {
        if (warp == 0)
            prefetch_tmap(&tmap_w);
        for (int slot = 0; slot < a.ring && ir < r_end; ++slot)
            issue(slot); // weights never depend on an earlier kernel: request them before the dependency wait
    }

    // ---- activations: everything below may depend on the kernel launched just before
    pdl_wait_prior_grid();
    if (a.x_qscale)
        build_records_half<NW>(a, rec_base, g_slice, n_groups, MT, kRec);
    else
    switch (a.x_bits) {
    case 1: build_records<1, NW>(a, rec_base, g_slice, n_groups, MT, kRec); break;
    case 2: build_records<2, NW>(a, rec_base, g_slice, n_groups, MT, kRec); break;
    case 3: build_records<3, NW>(a, rec_base, g_slice, n_groups, MT, kRec); break;
    case 4: build_records<4, NW>(a, rec_base, g_slice, n_groups, MT, kRec); break;
    case 5: build_records<5, NW>(a, rec_base, g_slice, n_groups, MT, kRec); break;
    case 6: build_records<6, NW>(a, rec_base, g_slice, n_groups, MT, kRec); break;
    case 7: build_records<7, NW>(a, rec_base, g_slice, n_groups, MT, kRec); break;
    default: build_records<8, NW>(a, rec_base, g_slice, n_groups, MT, kRec); break;
    }
    __syncthreads();

    const uint32_t flip = a.w_signed ? 0xffffffffu : 0u;
    const int zoff = a.w_signed ? (1 << (Q - 1)) : 0;
    const uint32_t swz = (uint32_t)((g >> 1) & 3); // 64B swizzle: 16-byte chunk index ^= (row >> 1) & 3
    int slot = 0;                                   // ring slot of the next stage this warp consumes
    uint32_t phase = 0;                             // parity of that slot's current use
    uint32_t round_parity = 0;
    bool ok = true;
    const int g_first = g_slice + st_begin * 4; // first 128-group of this warp's stage range
    const uint8_t *recs = rec_base + (size_t)st_begin * 4 * kRec;

    if (active) {
        for (int r = r_begin + ts; r < r_end; r += tiles_per_round, round_parity ^= 1) {
            const int n0 = r * 16;

            int acc[X::kSets][MT][4];
            float facc[MT][4];
            int xs[MT][2];
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
#pragma unroll
                    for (int k = 0; k < X::kSets; ++k)
                        acc[k][mt][e] = 0;
                    facc[mt][e] = 0.f;
                }
                xs[mt][0] = xs[mt][1] = 0;
            }

            // GROUP mode: lane l fetches scale and zero point of row l / 2 for the two groups (l & 1) * 2 + {0, 1} of a
            // stage, one stage ahead, packed as the fp32 bits of the scale (an fp16 value: its low 13 mantissa bits are
            // zero) with the zero point in the low byte; fold() gets the value it needs with one shuffle.
            uint32_t pk_cur[2] = { 0, 0 }, pk_next[2] = { 0, 0 };
            const bool row_ok = n0 + (lane >> 1) < a.N;
            const size_t row_off = (size_t)(n0 + (lane >> 1)) * a.scale_groups;
            auto fetch_scales = [&](int j, uint32_t (&pk)[2]) {
#pragma unroll
                for (int k = 0; k < 2; ++k) {
                    const int gg = g_first + j * 4 + (lane & 1) * 2 + k;
                    pk[k] = 0;
                    if (gg < a.total_groups && row_ok) {
                        const size_t idx = row_off + (GPS1 ? gg : gg / a.groups_per_scale);
                        uint32_t v = __float_as_uint(__half2float(ld_half(a.w_scale + idx)));
                        if (a.w_zero)
                            v |= (uint32_t)a.w_zero[idx];
                        pk[k] = v;
                    }
                }
            };
            if (GROUPED && my_nst > 0)
                fetch_scales(0, pk_next);
            bool pending = false; // GROUP mode: accumulators hold an unfinished scale group
            int pending_gi = 0;
            int in_group = GPS1 ? 0 : g_first % a.groups_per_scale; // 128-groups already seen of the current scale group

            // fold the integer accumulators of a finished scale group into fp32; gi = group within the stage.
            // v = acc0 + acc1 / 2^kShift - (zero + offset) * sum(x) is exact; with one scale group per 128 features its
            // magnitude is below 2^22 for the narrow bit widths, where int -> float is done with the 1.5 * 2^23 trick
            // (two ALU/FMA operations) instead of a conversion instruction.
            constexpr long long kBound = 128LL * (XU8 ? 255 : 128) * (((1 << Q) - 1) + ((1 << Q) - 1) + (1 << (Q - 1)));
            constexpr bool kMagic = GPS1 && kBound < (1LL << 22);
            auto fold = [&](int gi) {
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const uint32_t pk = __shfl_sync(0xffffffffu, (gi & 1) ? pk_cur[1] : pk_cur[0], 2 * (g + 8 * h) + (gi >> 1));
                    const float sc_w = __uint_as_float(pk & 0xffffff00u);
                    const int z = zoff + (int)(pk & 0xffu);
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
                        for (int j = 0; j < 2; ++j) {
                            int v = acc[0][mt][2 * h + j];
                            if (X::kSets == 2)
                                v += acc[X::kSets - 1][mt][2 * h + j] >> X::kShift;
                            v -= z * xs[mt][j];
                            const float fv = kMagic ? __int_as_float(v + 0x4b400000) - 12582912.0f : (float)v;
                            facc[mt][2 * h + j] = fmaf(fv, sc_w, facc[mt][2 * h + j]);
#pragma unroll
                            for (int k = 0; k < X::kSets; ++k)
                                acc[k][mt][2 * h + j] = 0;
                        }
                    }
                }
#pragma unroll
                for (int mt = 0; mt < MT; ++mt)
                    xs[mt][0] = xs[mt][1] = 0;
            };

            for (int j = 0; j < my_nst && ok; ++j) {
                if (GROUPED) {
                    pk_cur[0] = pk_next[0];
                    pk_cur[1] = pk_next[1];
                    if (j + 1 < my_nst)
                        fetch_scales(j + 1, pk_next);
                }
                ok = mbar_wait_bounded(&my_full[slot], phase, a.status, STATUS_TIMEOUT_TMA);
                if (!ok)
                    break;
                const uint8_t *stage = my_ring + (size_t)slot * kStageBytes;
                const int groups_here = min(4, a.total_groups - (g_first + j * 4));
#pragma unroll
                for (int gi = 0; gi < 4; ++gi) {
                    if (gi < groups_here) {
                        const uint32_t off = (((uint32_t)gi ^ swz) << 4) + (t << 2);
                        uint32_t pa[Q], pb[Q];
#pragma unroll
                        for (int b = 0; b < Q; ++b) {
                            pa[b] = *reinterpret_cast<const uint32_t *>(stage + b * 1024 + g * 64 + off);
                            pb[b] = *reinterpret_cast<const uint32_t *>(stage + b * 1024 + (g + 8) * 64 + off);
                        }
                        pa[Q - 1] ^= flip;
                        pb[Q - 1] ^= flip;
                        uint32_t ra[8], rb[8];
                        X::run(pa, ra);
                        X::run(pb, rb);
                        const uint8_t *rec = recs + (size_t)(j * 4 + gi) * kRec;
#pragma unroll
                        for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
                            for (int ip = 0; ip < 2; ++ip) {
                                const uint4 bf = *reinterpret_cast<const uint4 *>(rec + ((mt * 2 + ip) * 32 + lane) * 16);
                                mma_u8<XU8>(acc[X::set_of_step(2 * ip)][mt], ra[4 * ip], rb[4 * ip], ra[4 * ip + 1], rb[4 * ip + 1], bf.x,
                                            bf.y);
                                mma_u8<XU8>(acc[X::set_of_step(2 * ip + 1)][mt], ra[4 * ip + 2], rb[4 * ip + 2], ra[4 * ip + 3],
                                            rb[4 * ip + 3], bf.z, bf.w);
                            }
                        }
                        const int *sums = reinterpret_cast<const int *>(rec + 1024 * MT);
#pragma unroll
                        for (int mt = 0; mt < MT; ++mt) {
                            const int2 sv = *reinterpret_cast<const int2 *>(sums + 8 * mt + 2 * t);
                            xs[mt][0] += sv.x;
                            xs[mt][1] += sv.y;
                        }
                        if (GROUPED) {
                            if (GPS1) {
                                fold(gi);
                            } else {
                                pending = true;
                                pending_gi = gi;
                                if (++in_group == a.groups_per_scale) {
                                    in_group = 0;
                                    fold(gi);
                                    pending = false;
                                }
                            }
                        }
                    }
                }
                // a scale group that continues in the next stage is folded with the scale staged for this one (the fold
                // is linear); after this point pk_cur is overwritten
                if (GROUPED && !GPS1 && pending) {
                    fold(pending_gi);
                    pending = false;
                }
                __syncwarp();
                if (lane == 0 && ir < r_end)
                    issue(slot); // the slot just consumed is free again
                if (++slot == a.ring) {
                    slot = 0;
                    phase ^= 1;
                }
            }
            __syncwarp();

            // ---- this warp's share of the tile: fp32 (GROUP) or exact int32, rows g, g + 8, tokens 8 mt + 2 t + {0, 1}
            int v[MT][4];
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    if (GROUPED) {
                        v[mt][e] = __float_as_int(facc[mt][e]);
                    } else {
                        int z = zoff;
                        const int n = n0 + g + 8 * (e >> 1);
                        if (a.scale_mode == ABQ_SCALE_CHANNEL && a.w_zero && n < a.N)
                            z += a.w_zero[n];
                        int x = acc[0][mt][e];
                        if (X::kSets == 2)
                            x += acc[X::kSets - 1][mt][e] >> X::kShift; // exact: every term of that set is a multiple of 2^kShift
                        v[mt][e] = x - z * xs[mt][e & 1];
                    }
                }
            }

            // ---- the warps of a tile meet in shared memory; part 0 adds the others in part order
            if (a.split > 1) {
                if (sc != 0) {
                    if (ok)
                        ok = mbar_wait_bounded(&red_free[ts], round_parity ^ 1, a.status, STATUS_TIMEOUT_PIPE); // previous round read
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                        for (int e = 0; e < 4; ++e)
                            red[(warp * 4 * MT + mt * 4 + e) * 32 + lane] = v[mt][e];
                    __syncwarp();
                    if (lane == 0)
                        mbar_arrive(&red_ready[ts]);
                    continue;
                }
                if (ok)
                    ok = mbar_wait_bounded(&red_ready[ts], round_parity, a.status, STATUS_TIMEOUT_PIPE);
                for (int k = 1; k < a.split; ++k) {
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const int pv = red[((warp + k) * 4 * MT + mt * 4 + e) * 32 + lane];
                            v[mt][e] = GROUPED ? __float_as_int(__int_as_float(v[mt][e]) + __int_as_float(pv)) : v[mt][e] + pv;
                        }
                }
                __syncwarp();
                if (lane == 0)
                    mbar_arrive(&red_free[ts]);
            }

            // ---- K split over CTAs as well: workspace slot per slice, last arrival adds them in slice order
            bool finish = true;
            if (a.slices > 1) {
                int *pslot = a.partials + ((size_t)s * a.tiles + r) * (size_t)a.M * 16;
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int tok = 8 * mt + 2 * t + (e & 1);
                        if (tok < a.M)
                            pslot[tok * 16 + g + 8 * (e >> 1)] = v[mt][e];
                    }
                }
                __threadfence();
                __syncwarp();
                int old = 0;
                if (lane == 0)
                    old = atomicAdd(a.counters + r, 1);
                old = __shfl_sync(0xffffffffu, old, 0);
                finish = old == a.slices - 1;
                if (finish) {
                    __threadfence();
                    if (lane == 0)
                        a.counters[r] = 0; // leave the counter ready for the next launch
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const int tok = 8 * mt + 2 * t + (e & 1);
                            int isum = 0;
                            float fsum = 0.f;
                            if (tok < a.M) {
                                for (int sl = 0; sl < a.slices; ++sl) { // fixed order: the result does not depend on who finishes
                                    const int pv =
                                        __ldcg(a.partials + ((size_t)sl * a.tiles + r) * (size_t)a.M * 16 + tok * 16 + g + 8 * (e >> 1));
                                    if (GROUPED)
                                        fsum += __int_as_float(pv);
                                    else
                                        isum += pv;
                                }
                            }
                            v[mt][e] = GROUPED ? __float_as_int(fsum) : isum;
                        }
                    }
                }
            }
            if (finish) {
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int tok = 8 * mt + 2 * t + (e & 1);
                        const int n = n0 + g + 8 * (e >> 1);
                        if (tok < a.M && n < a.N) {
                            const size_t o = (size_t)tok * a.N + n;
                            if (a.out_dtype == ABQ_OUT_INT32) {
                                reinterpret_cast<int *>(a.D)[o] = v[mt][e];
                            } else {
                                __half h;
                                if (a.scale_mode == ABQ_SCALE_TENSOR_COMPAT) {
                                    h = __hmul(__int2half_rn(v[mt][e]), ld_half(a.C));
                                } else {
                                    float f = GROUPED ? __int_as_float(v[mt][e]) : (float)v[mt][e] * __half2float(ld_half(a.w_scale + n));
                                    if (a.x_scale)
                                        f *= a.x_scale[tok];
                                    h = __float2half_rn(f);
                                }
                                if (a.residual)
                                    h = __hadd(h, a.residual[o]);
                                reinterpret_cast<__half *>(a.D)[o] = h;
                            }
                        }
                    }
                }
            }
        }
    }

    // A wait that expired may have left copies in flight: give them one more bounded chance to land before the
    // shared memory they target is released.
    if (!ok && lane == 0) {
        for (int i = 0; i < a.ring; ++i)
            mbar_wait_bounded(&my_full[i], 0, nullptr, 0);
    }
}

// ------------------------------------------------------------------------------------------- host side

template <int Q, int MT, bool XU8, int NW>
static cudaError_t launch_variant(const abq_gemm_state *st, const DecodeArgs &args, cudaStream_t stream)
{
    const int grouped = args.scale_mode != ABQ_SCALE_GROUP ? 0 : (args.groups_per_scale == 1 ? 1 : 2);
    auto kern = grouped == 0 ? decode_kernel<Q, MT, XU8, false, true, NW>
                             : (grouped == 1 ? decode_kernel<Q, MT, XU8, true, true, NW> : decode_kernel<Q, MT, XU8, true, false, NW>);
    static thread_local SmemOptIn opted[3]; // per instantiation, scale mode and host thread
    {
        cudaError_t e = opted[grouped].ensure(kern, st->shared_mem_size);
        if (e != cudaSuccess)
            return e;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(st->grid[0], 1, 1);
    cfg.blockDim = dim3(NW * 32);
    cfg.dynamicSmemBytes = st->shared_mem_size;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    int na = 0;
    if (st->p.flags & ABQ_FLAG_PDL) {
        attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[na].val.programmaticStreamSerializationAllowed = 1;
        ++na;
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
    CUtensorMap tm; // the plan stores the descriptor as plain words: copy to a correctly aligned object
    memcpy(&tm, st->tmap[0], sizeof(tm));
    return cudaLaunchKernelEx(&cfg, kern, tm, args);
}

template <int Q>
static cudaError_t launch_q(const abq_gemm_state *st, const DecodeArgs &args, int MT, bool xu8, cudaStream_t stream)
{
    if (st->block[0] == 16 * 32) {
        if (MT == 1)
            return xu8 ? launch_variant<Q, 1, true, 16>(st, args, stream) : launch_variant<Q, 1, false, 16>(st, args, stream);
        return xu8 ? launch_variant<Q, 2, true, 16>(st, args, stream) : launch_variant<Q, 2, false, 16>(st, args, stream);
    }
    if (MT == 1)
        return xu8 ? launch_variant<Q, 1, true, 8>(st, args, stream) : launch_variant<Q, 1, false, 8>(st, args, stream);
    return xu8 ? launch_variant<Q, 2, true, 8>(st, args, stream) : launch_variant<Q, 2, false, 8>(st, args, stream);
}


// one definition per weight width, in gemm_decode_w<Q>.cu
#define ABQ_DECODE_WIDTH(Q)                                                                                                            \
    cudaError_t decode_launch_w##Q(const abq_gemm_state *st, const DecodeArgs &args, int MT, bool xu8, cudaStream_t stream)           \
    {                                                                                                                                  \
        return launch_q<Q>(st, args, MT, xu8, stream);                                                                                 \
    }
cudaError_t decode_launch_w1(const abq_gemm_state *st, const DecodeArgs &args, int MT, bool xu8, cudaStream_t stream);
cudaError_t decode_launch_w2(const abq_gemm_state *st, const DecodeArgs &args, int MT, bool xu8, cudaStream_t stream);
cudaError_t decode_launch_w3(const abq_gemm_state *st, const DecodeArgs &args, int MT, bool xu8, cudaStream_t stream);
cudaError_t decode_launch_w4(const abq_gemm_state *st, const DecodeArgs &args, int MT, bool xu8, cudaStream_t stream);
cudaError_t decode_launch_w5(const abq_gemm_state *st, const DecodeArgs &args, int MT, bool xu8, cudaStream_t stream);
cudaError_t decode_launch_w6(const abq_gemm_state *st, const DecodeArgs &args, int MT, bool xu8, cudaStream_t stream);
cudaError_t decode_launch_w7(const abq_gemm_state *st, const DecodeArgs &args, int MT, bool xu8, cudaStream_t stream);
cudaError_t decode_launch_w8(const abq_gemm_state *st, const DecodeArgs &args, int MT, bool xu8, cudaStream_t stream);

} // namespace abq
