// Decode-shape GEMM (M <= 16), route ABQ_ROUTE_I8_MMA.
//
// HBM-bound: every weight plane word is read exactly once, and the kernel is organised so that the
// SM never waits for a CTA-wide event while planes are in flight.
//
//  * Work unit = 16 weight rows x one K-slice.  The grid is persistent (one or two CTAs per SM); CTA i
//    owns a contiguous range of units, and each of its eight warps walks that range with stride 8.
//  * Every warp feeds itself: lane 0 issues 3-D TMA boxes (all q planes x 16 rows x 512 input features,
//    64-byte rows, 64B-swizzled) into a warp-private ring and refills a slot right after the warp has
//    consumed it, across unit boundaries, so the stream never drains before the kernel ends.
//  * A thread takes one 32-bit word per plane and row and recombines the q plane words into byte codes
//    with a butterfly (expand.cuh); the bytes are the A operand of mma.sync.m16n8k32 (u8 x s8/u8 -> s32).
//    Two accumulator sets carry different power-of-two scales, which saves the shifts that would
//    otherwise normalise the bit fields.
//  * The B operand (tokens) comes from activation records prepared once per GEMM (xprep.cu).
//  * Scale / zero-point dequantisation is fused: per scale group the int32 accumulators are folded into
//    fp32; scales and zero points are fetched one stage ahead and handed round by shuffles.
//  * Split-K partials go to a workspace slot per slice; the warp that arrives last at a tile's counter
//    adds the slots in slice order (deterministic) and writes the output.
//
// Covers what the reference does with plane-stacked 1-bit MMAs and an smem shift-accumulate epilogue
// (engine/mma_any/aq_bmma_kernel.h:109-271, 485-580) and with its fp16 scalar-scale epilogue
// (fastertransformer/.../abqgemm/mma_any/aq_bmma_kernel.h:474-524).
#include <cuda.h>
#include <cstring>

#include "abq_common.cuh"
#include "abq_kernels.h"
#include "expand.cuh"

namespace abq {

constexpr int kMaxRing = 6;
constexpr int kMaxWarps = 16;

struct DecodeArgs {
    int M, N, K;
    int tiles;            // ceil(N / 16)
    int total_groups;     // K / 128
    int stages_per_slice; // 512-feature stages per K-slice
    int slices;           // split-K factor; the grid is slices * ctas_per_slice
    int ctas_per_slice;
    int ring;             // TMA stages per warp
    const uint8_t *records;
    int *counters;        // one per tile, zeroed by xprep_decode
    int *partials;        // [slice][tile][token][16 rows] int32 or fp32 bit patterns
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
};

// NW warps per CTA, one CTA per SM.  CTA b works on K-slice b / ctas_per_slice and on an even share of the
// 16-row tiles; its warps take those tiles with stride NW.
template <int Q, int MT, bool XU8, bool GROUPED, bool GPS1, int NW>
__global__ void __launch_bounds__(NW * 32, 1) decode_kernel(const __grid_constant__ CUtensorMap tmap_w, const DecodeArgs a)
{
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    constexpr int kStageBytes = Q * 1024; // [plane][16 rows][64 B]
    constexpr int kRec = decode_record_bytes(MT);
    using X = Expand<Q>;
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t *ring_base = smem;
    uint8_t *rec_base = ring_base + (size_t)NW * a.ring * kStageBytes;
    uint64_t *bars = reinterpret_cast<uint64_t *>(rec_base + (size_t)a.stages_per_slice * 4 * kRec);
    uint64_t *full = bars;                   // [warp][slot]
    uint64_t *recbar = bars + NW * kMaxRing; // activation records of this CTA's slice

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int s = blockIdx.x / a.ctas_per_slice;      // K-slice of this CTA
    const int cb = blockIdx.x - s * a.ctas_per_slice; // position among the CTAs of the slice
    const int r_begin = (int)((long long)cb * a.tiles / a.ctas_per_slice);
    const int r_end = (int)((long long)(cb + 1) * a.tiles / a.ctas_per_slice);
    const int total_stages = (a.total_groups + 3) >> 2;
    const int nst = max(0, min(total_stages - s * a.stages_per_slice, a.stages_per_slice)); // stages of this slice
    const int g_first = s * a.stages_per_slice * 4;                                          // its first 128-group
    const int n_groups = max(0, min(a.total_groups - g_first, a.stages_per_slice * 4));

    if (threadIdx.x == 0) {
        for (int w = 0; w < NW; ++w)
            for (int i = 0; i < a.ring; ++i)
                mbar_init(&full[w * kMaxRing + i], 1);
        mbar_init(recbar, 1);
        fence_mbar_init();
    }
    __syncthreads();
    pdl_launch_dependents();

    // ---- request side (lane 0 of every warp): cursor over (tile, stage) in the order the warp consumes them
    int ir = r_begin + warp, ij = 0;
    uint8_t *my_ring = ring_base + (size_t)warp * a.ring * kStageBytes;
    uint64_t *my_full = full + warp * kMaxRing;
    auto issue = [&](int slot) {
        mbar_arrive_expect_tx(&my_full[slot], kStageBytes);
        tma_load_3d(my_ring + (size_t)slot * kStageBytes, &tmap_w, (s * a.stages_per_slice + ij) * 16, ir * 16, 0, &my_full[slot]);
        if (++ij == nst) {
            ij = 0;
            ir += NW;
        }
    };
    if (lane == 0 && nst > 0) {
        if (warp == 0)
            prefetch_tmap(&tmap_w);
        for (int slot = 0; slot < a.ring && ir < r_end; ++slot)
            issue(slot); // weights never depend on an earlier kernel: request them before the dependency wait
    }
    if (threadIdx.x == 0) {
        pdl_wait_prior_grid(); // records, counters and partial slots belong to the kernel launched just before
        if (n_groups > 0) {
            mbar_arrive_expect_tx(recbar, (uint32_t)(n_groups * kRec));
            bulk_load(rec_base, a.records + (size_t)g_first * kRec, (uint32_t)(n_groups * kRec), recbar);
        } else {
            mbar_arrive(recbar);
        }
    }
    __syncwarp();

    const uint32_t flip = a.w_signed ? 0xffffffffu : 0u;
    const int zoff = a.w_signed ? (1 << (Q - 1)) : 0;
    const uint32_t swz = (uint32_t)((g >> 1) & 3); // 64B swizzle: 16-byte chunk index ^= (row >> 1) & 3
    int slot = 0;                                   // ring slot of the next stage this warp consumes
    uint32_t phase = 0;                             // parity of that slot's current use

    bool ok = mbar_wait_bounded(recbar, 0, a.status, STATUS_TIMEOUT_TMA);
    const uint8_t *recs = rec_base;

    for (int r = r_begin + warp; r < r_end; r += NW) {
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

        // GROUP mode: lane l fetches scale and zero point of row l / 2 for the two groups (l & 1) * 2 + {0, 1} of a stage,
        // one stage ahead, packed as the fp32 bits of the scale (an fp16 value: its low 13 mantissa bits are zero) with
        // the zero point in the low byte; fold() gets the value it needs with one shuffle.
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
        if (GROUPED && nst > 0)
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
                const float sc = __uint_as_float(pk & 0xffffff00u);
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
                        facc[mt][2 * h + j] = fmaf(fv, sc, facc[mt][2 * h + j]);
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

        for (int j = 0; j < nst && ok; ++j) {
            if (GROUPED) {
                pk_cur[0] = pk_next[0];
                pk_cur[1] = pk_next[1];
                if (j + 1 < nst)
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
                            mma_u8<XU8>(acc[X::set_of_step(2 * ip)][mt], ra[4 * ip], rb[4 * ip], ra[4 * ip + 1], rb[4 * ip + 1], bf.x, bf.y);
                            mma_u8<XU8>(acc[X::set_of_step(2 * ip + 1)][mt], ra[4 * ip + 2], rb[4 * ip + 2], ra[4 * ip + 3], rb[4 * ip + 3], bf.z,
                                        bf.w);
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
            // a scale group that continues in the next stage is folded with the scale staged for this one (the fold is
            // linear); after this point pk_cur is overwritten
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

        // ---- unit result: fp32 (GROUP) or exact int32 for rows g, g + 8 and tokens 8 mt + 2 t + {0, 1}
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

        bool finish = true;
        if (a.slices > 1) {
            int *slot = a.partials + ((size_t)s * a.tiles + r) * (size_t)a.M * 16;
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int tok = 8 * mt + 2 * t + (e & 1);
                    if (tok < a.M)
                        slot[tok * 16 + g + 8 * (e >> 1)] = v[mt][e];
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
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int tok = 8 * mt + 2 * t + (e & 1);
                        int isum = 0;
                        float fsum = 0.f;
                        if (tok < a.M) {
                            for (int sl = 0; sl < a.slices; ++sl) { // fixed order: the result does not depend on who finishes
                                const int pv = __ldcg(a.partials + ((size_t)sl * a.tiles + r) * (size_t)a.M * 16 + tok * 16 + g + 8 * (e >> 1));
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
                            reinterpret_cast<__half *>(a.D)[o] = h;
                        }
                    }
                }
            }
        }
    }

    // A wait that expired may have left copies in flight: give them one more bounded chance to land before the
    // shared memory they target is released.
    if (!ok && lane == 0) {
        for (int slot = 0; slot < a.ring; ++slot)
            mbar_wait_bounded(&my_full[slot], 0, nullptr, 0);
    }
}

// ------------------------------------------------------------------------------------------- host side

struct DecodeLayout {
    int MT, NW, tiles, total_groups, slices, stages_per_slice, ctas_per_slice, ring;
    size_t smem, off_counters, off_partials, bytes;
};

static int device_sms()
{
    int dev = 0, v = 0;
    if (cudaGetDevice(&dev) == cudaSuccess && cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && v > 0)
        return v;
    return 148;
}

// Workspace: [activation records][tile counters][split-K partial slots for up to kDecodeMaxSlices slices]
static void workspace_layout(int M, int N, int K, size_t *off_counters, size_t *off_partials, size_t *total)
{
    const int MT = M <= 8 ? 1 : 2;
    const size_t rec = (size_t)(K / 128) * decode_record_bytes(MT);
    const int tiles = (N + 15) / 16;
    *off_counters = (rec + 255) & ~(size_t)255;
    *off_partials = (*off_counters + (size_t)tiles * 4 + 255) & ~(size_t)255;
    *total = *off_partials + (size_t)kDecodeMaxSlices * tiles * M * 16 * 4;
}

size_t decode_workspace_bytes(int M, int N, int K)
{
    size_t a, b, total;
    workspace_layout(M, N, K, &a, &b, &total);
    return total;
}

// Tile shape of a launch: warps per CTA, split-K factor, ring depth.  One CTA per SM; the split is chosen so that
// every warp of the machine gets about one 16-row tile of its slice (the kernel is latency-bound per warp, so
// equal tile counts per warp matter more than long slices).
static bool make_layout(const abq_gemm_params &p, DecodeLayout *L)
{
    const int Q = p.w_bits;
    L->MT = p.M <= 8 ? 1 : 2;
    L->tiles = (p.N + 15) / 16;
    L->total_groups = p.K / 128;
    const int total_stages = (L->total_groups + 3) / 4;
    const int sms = device_sms();
    const int stage_bytes = Q * 1024;
    const int rec = decode_record_bytes(L->MT);
    const int want_nw = env_int("ABQ_DECODE_WARPS", 16);
    for (int nw = want_nw; nw >= 8; nw -= 8) {
        int slices = (nw * sms + L->tiles / 2) / L->tiles;
        slices = slices < 1 ? 1 : slices;
        slices = slices > kDecodeMaxSlices ? kDecodeMaxSlices : slices;
        slices = slices > total_stages ? total_stages : slices;
        slices = env_int("ABQ_DECODE_SLICES", slices);
        if (slices < 1 || slices > kDecodeMaxSlices || slices > total_stages)
            return false;
        const int sps = (total_stages + slices - 1) / slices;
        slices = (total_stages + sps - 1) / sps; // drop slices that would be empty
        int cps = sms / slices;
        cps = cps > L->tiles ? L->tiles : cps;
        cps = cps < 1 ? 1 : cps;
        const size_t fixed = 1024 + (size_t)sps * 4 * rec + ((size_t)nw * kMaxRing + 1) * 8;
        const size_t budget = 226 * 1024;
        if (fixed >= budget)
            continue;
        int ring = (int)((budget - fixed) / ((size_t)nw * stage_bytes));
        ring = ring > kMaxRing ? kMaxRing : ring;
        ring = env_int("ABQ_DECODE_RING", ring);
        if (ring < 2 && nw > 8)
            continue;
        if (ring < 1 || ring > kMaxRing)
            return false;
        L->NW = nw;
        L->slices = slices;
        L->stages_per_slice = sps;
        L->ctas_per_slice = cps;
        L->ring = ring;
        L->smem = fixed + (size_t)nw * ring * stage_bytes;
        workspace_layout(p.M, p.N, p.K, &L->off_counters, &L->off_partials, &L->bytes);
        return L->smem <= 227 * 1024;
    }
    return false;
}

template <int Q, int MT, bool XU8, int NW>
static cudaError_t launch_variant(const abq_gemm_state *st, const DecodeArgs &args, cudaStream_t stream)
{
    const int grouped = args.scale_mode != ABQ_SCALE_GROUP ? 0 : (args.groups_per_scale == 1 ? 1 : 2);
    auto kern = grouped == 0 ? decode_kernel<Q, MT, XU8, false, true, NW>
                             : (grouped == 1 ? decode_kernel<Q, MT, XU8, true, true, NW> : decode_kernel<Q, MT, XU8, true, false, NW>);
    static thread_local size_t configured[3] = { 0, 0, 0 }; // per instantiation and thread: largest size already opted in
    if (st->shared_mem_size > configured[grouped]) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)st->shared_mem_size);
        if (e != cudaSuccess)
            return e;
        configured[grouped] = st->shared_mem_size;
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
static cudaError_t launch_q(const abq_gemm_state *st, const DecodeArgs &args, int MT, bool xu8, int nw, cudaStream_t stream)
{
    if (nw == 16) {
        if (MT == 1)
            return xu8 ? launch_variant<Q, 1, true, 16>(st, args, stream) : launch_variant<Q, 1, false, 16>(st, args, stream);
        return xu8 ? launch_variant<Q, 2, true, 16>(st, args, stream) : launch_variant<Q, 2, false, 16>(st, args, stream);
    }
    if (MT == 1)
        return xu8 ? launch_variant<Q, 1, true, 8>(st, args, stream) : launch_variant<Q, 1, false, 8>(st, args, stream);
    return xu8 ? launch_variant<Q, 2, true, 8>(st, args, stream) : launch_variant<Q, 2, false, 8>(st, args, stream);
}

abq_status decode_plan(abq_gemm_state *st)
{
    const abq_gemm_params &p = st->p;
    if (p.M > 16)
        return ABQ_ERR_UNSUPPORTED;
    if (p.scale_mode == ABQ_SCALE_GROUP && (p.group_size % 128 != 0))
        return ABQ_ERR_UNSUPPORTED;
    DecodeLayout L;
    if (!make_layout(p, &L))
        return ABQ_ERR_UNSUPPORTED;
    if (!p.workspace || p.workspace_bytes < L.bytes)
        return ABQ_ERR_WORKSPACE;

    const uint64_t KW = (uint64_t)p.K / 32;
    const uint64_t dims[3] = { KW, (uint64_t)p.N, (uint64_t)p.w_bits };
    const uint64_t strides[2] = { KW * 4, KW * 4 * (uint64_t)p.N };
    const uint32_t box[3] = { 16, 16, (uint32_t)p.w_bits };
    if (!encode_tmap(st->tmap[0], TMAP_U32, 3, p.W, dims, strides, box, TMAP_SWIZZLE_64B))
        return ABQ_ERR_CUDA;

    st->grid[0] = L.slices * L.ctas_per_slice;
    st->grid[1] = st->grid[2] = 1;
    st->block[0] = L.NW * 32;
    st->block[1] = st->block[2] = 1;
    st->cluster = L.slices;
    st->shared_mem_size = L.smem;
    st->tile[0] = L.stages_per_slice;
    st->tile[1] = L.ring;
    st->tile[2] = L.ctas_per_slice;
    st->tile[3] = L.MT;
    return ABQ_OK;
}

cudaError_t decode_launch(const abq_gemm_state *st, cudaStream_t stream)
{
    const abq_gemm_params &p = st->p;
    const int MT = st->tile[3];
    const bool pdl = (p.flags & ABQ_FLAG_PDL) != 0;
    size_t off_counters, off_partials, total;
    workspace_layout(p.M, p.N, p.K, &off_counters, &off_partials, &total);
    uint8_t *ws = reinterpret_cast<uint8_t *>(p.workspace);
    const int tiles = (p.N + 15) / 16;
    cudaError_t e = cudaSuccess;
    if (!env_int("ABQ_EXPERIMENT_SKIP_XPREP", 0))
        e = xprep_decode(reinterpret_cast<const uint32_t *>(p.X), ws, reinterpret_cast<int *>(ws + off_counters), tiles, p.M, p.K,
                         p.x_bits, p.x_signed, MT, pdl, stream);
    if (e != cudaSuccess)
        return e;
    DecodeArgs a;
    a.M = p.M;
    a.N = p.N;
    a.K = p.K;
    a.tiles = tiles;
    a.total_groups = p.K / 128;
    a.stages_per_slice = st->tile[0];
    a.slices = st->cluster;
    a.ctas_per_slice = st->tile[2];
    a.ring = st->tile[1];
    a.records = ws;
    a.counters = reinterpret_cast<int *>(ws + off_counters);
    a.partials = reinterpret_cast<int *>(ws + off_partials);
    a.D = p.D;
    a.w_scale = reinterpret_cast<const __half *>(p.w_scale);
    a.w_zero = p.w_zero;
    a.x_scale = p.x_scale;
    a.C = reinterpret_cast<const __half *>(p.C);
    a.out_dtype = p.out_dtype;
    a.scale_mode = p.scale_mode;
    a.groups_per_scale = p.scale_mode == ABQ_SCALE_GROUP ? p.group_size / 128 : 1;
    a.scale_groups = p.scale_mode == ABQ_SCALE_GROUP ? p.K / p.group_size : 1;
    a.w_signed = p.w_signed;
    a.status = p.status_word;
    const bool xu8 = !p.x_signed && p.x_bits == 8;
    switch (p.w_bits) {
    case 1: return launch_q<1>(st, a, MT, xu8, st->block[0] / 32, stream);
    case 2: return launch_q<2>(st, a, MT, xu8, st->block[0] / 32, stream);
    case 3: return launch_q<3>(st, a, MT, xu8, st->block[0] / 32, stream);
    case 4: return launch_q<4>(st, a, MT, xu8, st->block[0] / 32, stream);
    case 5: return launch_q<5>(st, a, MT, xu8, st->block[0] / 32, stream);
    case 6: return launch_q<6>(st, a, MT, xu8, st->block[0] / 32, stream);
    case 7: return launch_q<7>(st, a, MT, xu8, st->block[0] / 32, stream);
    case 8: return launch_q<8>(st, a, MT, xu8, st->block[0] / 32, stream);
    default: return cudaErrorInvalidValue;
    }
}

} // namespace abq
