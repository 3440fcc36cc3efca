// Decode-shape GEMM (M <= 16), route ABQ_ROUTE_I8_MMA.
//
// HBM-bound: the weight bit-planes are streamed exactly once.  Per CTA a producer warp drives a ring
// of TMA stages (one 3-D box = all q planes x 64 weight rows x 1024 input features, 128-byte rows,
// 128B-swizzled); four consumer warps each own 16 weight rows.  A consumer thread takes one 32-bit word
// per plane and row, recombines the q plane words into eight registers of unsigned byte codes
// (planes_to_bytes) and feeds them as the A operand of mma.sync.m16n8k32 (u8 x s8/u8 -> s32); the B
// operand (up to 8 tokens per MMA) comes from activation records prepared once per GEMM by
// xprep_decode, whose byte order matches the expansion.  The input-feature range is split over the
// CTAs of a thread-block cluster (split-K); partial sums are reduced through distributed shared
// memory in rank order, so the result does not depend on scheduling.  Scale / zero-point
// dequantisation is fused: per scale group the int32 accumulators are folded into fp32.
//
// Covers what the reference does with plane-stacked 1-bit MMAs and an smem shift-accumulate epilogue
// (engine/mma_any/aq_bmma_kernel.h:109-271, 485-580) and with its fp16 scalar-scale epilogue
// (fastertransformer/.../abqgemm/mma_any/aq_bmma_kernel.h:474-524).
#include <cuda.h>
#include <cstring>

#include "abq_common.cuh"
#include "abq_kernels.h"

namespace abq {

constexpr int kConsumerWarps = kDecodeBN / 16;
constexpr int kDecodeThreads = (kConsumerWarps + 1) * 32;
constexpr int kMaxStages = 8;
constexpr int kScaleStageWords = 2 * 2 * 16 * 8; // per consumer warp: two buffers of 16 rows x 8 groups, scales and zero points

struct DecodeArgs {
    int M, N, K;
    int chunks_per_cta;  // pipeline chunks (1024 features each) per CTA; blockIdx.y selects the slice
    int stages;
    int rec_smem_bytes;  // shared memory reserved for the activation records of one slice
    const uint8_t *records;
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

template <int Q, int MT, bool XU8>
__global__ void __launch_bounds__(kDecodeThreads) decode_kernel(const __grid_constant__ CUtensorMap tmap_w, const DecodeArgs a)
{
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    constexpr int kStageBytes = Q * kDecodeBN * 128;
    constexpr int kRec = decode_record_bytes(MT);
    // carve-up: [stages][records][reduce buffer][barriers]
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t *stage_base = smem;
    uint8_t *rec_base = stage_base + (size_t)a.stages * kStageBytes;
    int *red = reinterpret_cast<int *>(rec_base + a.rec_smem_bytes);
    float *scale_stage = reinterpret_cast<float *>(red + kDecodeBN * 8 * MT); // [warp][buffer][16 rows][8 groups] scale, then zero
    uint64_t *bars = reinterpret_cast<uint64_t *>(scale_stage + kConsumerWarps * kScaleStageWords);
    uint64_t *full = bars, *empty = bars + kMaxStages, *xbar = bars + 2 * kMaxStages;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = blockIdx.x * kDecodeBN;
    const int total_groups = a.K >> 7;
    const int g_begin = blockIdx.y * a.chunks_per_cta * 8;                          // first 128-group of this slice
    const int g_count = max(0, min(total_groups - g_begin, a.chunks_per_cta * 8));   // groups in this slice
    const int n_chunks = (g_count + 7) >> 3;

    if (threadIdx.x == 0) {
        for (int s = 0; s < a.stages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], kConsumerWarps);
        }
        mbar_init(xbar, 1);
        fence_mbar_init();
    }
    __syncthreads();
    pdl_launch_dependents();

    if (warp == kConsumerWarps) {
        // ---------------- producer warp: weights first (they never depend on an earlier kernel)
        if (lane == 0) {
            prefetch_tmap(&tmap_w);
            int c = 0;
            const int prologue = min(n_chunks, a.stages);
            for (; c < prologue; ++c) {
                mbar_arrive_expect_tx(&full[c], kStageBytes);
                tma_load_3d(stage_base + (size_t)c * kStageBytes, &tmap_w, (g_begin + c * 8) * 4, n0, 0, &full[c]);
            }
            pdl_wait_prior_grid(); // activation records are written by the kernel launched just before
            if (g_count > 0) {
                mbar_arrive_expect_tx(xbar, (uint32_t)(g_count * kRec));
                bulk_load(rec_base, a.records + (size_t)g_begin * kRec, (uint32_t)(g_count * kRec), xbar);
            } else {
                mbar_arrive(xbar);
            }
            for (; c < n_chunks; ++c) {
                const int s = c % a.stages;
                const uint32_t parity = ((c / a.stages) - 1) & 1;
                if (!mbar_wait_bounded(&empty[s], parity, a.status, STATUS_TIMEOUT_PIPE))
                    break;
                mbar_arrive_expect_tx(&full[s], kStageBytes);
                tma_load_3d(stage_base + (size_t)s * kStageBytes, &tmap_w, (g_begin + c * 8) * 4, n0, 0, &full[s]);
            }
        }
        __syncwarp();
    } else {
        // ---------------- consumer warps
        const int g = lane >> 2, t = lane & 3;
        const int row_a = warp * 16 + g; // tile-local weight rows of this thread: row_a and row_a + 8
        const bool grouped = a.scale_mode == ABQ_SCALE_GROUP;
        const int zoff = a.w_signed ? (1 << (Q - 1)) : 0;
        int acc[MT][4];
        float facc[MT][4];
        int xs[MT][2];
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                acc[mt][e] = 0;
                facc[mt][e] = 0.f;
            }
            xs[mt][0] = xs[mt][1] = 0;
        }
        // GROUP mode: the scales / zero points of a chunk (16 rows x 8 groups per warp) are fetched one chunk ahead
        // into registers (lane = row * 2 + half, four groups each) and parked in a warp-private staging buffer, so
        // that folding a group never waits on global memory.
        float *sc_stage = scale_stage + warp * kScaleStageWords;
        int *z_stage = reinterpret_cast<int *>(sc_stage + 2 * 16 * 8);
        float pre_sc[4];
        int pre_z[4];
        auto prefetch_scales = [&](int c) {
            const int n = n0 + warp * 16 + (lane >> 1);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int gl = c * 8 + (lane & 1) * 4 + j;
                pre_sc[j] = 0.f;
                pre_z[j] = 0;
                if (grouped && gl < g_count && n < a.N) {
                    const size_t idx = (size_t)n * a.scale_groups + (g_begin + gl) / a.groups_per_scale;
                    pre_sc[j] = __half2float(ld_half(a.w_scale + idx));
                    if (a.w_zero)
                        pre_z[j] = a.w_zero[idx];
                }
            }
        };
        auto park_scales = [&](int c) {
            float *sdst = sc_stage + (c & 1) * 128 + (lane >> 1) * 8 + (lane & 1) * 4;
            int *zdst = z_stage + (c & 1) * 128 + (lane >> 1) * 8 + (lane & 1) * 4;
            *reinterpret_cast<float4 *>(sdst) = make_float4(pre_sc[0], pre_sc[1], pre_sc[2], pre_sc[3]);
            *reinterpret_cast<int4 *>(zdst) = make_int4(pre_z[0], pre_z[1], pre_z[2], pre_z[3]);
            __syncwarp();
        };
        if (grouped)
            prefetch_scales(0);
        bool ok = mbar_wait_bounded(xbar, 0, a.status, STATUS_TIMEOUT_TMA);
        int pending_gi = -1; // group (within the current chunk) whose scale group still has unfolded accumulators

        // One scale group finished: fold the integer accumulators into fp32 (GROUP mode).  `buf`/`gi` select the
        // staged scale and zero point of the 128-group that closes it.
        auto fold = [&](int buf, int gi) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const float sc = sc_stage[buf * 128 + (g + 8 * h) * 8 + gi];
                const int z = zoff + z_stage[buf * 128 + (g + 8 * h) * 8 + gi];
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
                    for (int j = 0; j < 2; ++j) {
                        const int v = acc[mt][2 * h + j] - z * xs[mt][j];
                        facc[mt][2 * h + j] = fmaf((float)v, sc, facc[mt][2 * h + j]);
                        acc[mt][2 * h + j] = 0;
                    }
                }
            }
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
                xs[mt][0] = xs[mt][1] = 0;
        };

        for (int c = 0; c < n_chunks && ok; ++c) {
            const int s = c % a.stages;
            ok = mbar_wait_bounded(&full[s], (c / a.stages) & 1, a.status, STATUS_TIMEOUT_TMA);
            if (!ok)
                break;
            const uint8_t *stage = stage_base + (size_t)s * kStageBytes;
            const int groups_here = min(8, g_count - c * 8);
            if (grouped) {
                park_scales(c);
                if (c + 1 < n_chunks)
                    prefetch_scales(c + 1);
            }
            for (int gi = 0; gi < groups_here; ++gi) {
                const int gl = c * 8 + gi; // group index inside the slice
                uint32_t pa[Q], pb[Q];
                const uint32_t off = (uint32_t)(((gi ^ g) << 4) + (t << 2)); // 128B swizzle: chunk ^= row & 7
#pragma unroll
                for (int b = 0; b < Q; ++b) {
                    const uint8_t *plane = stage + b * (kDecodeBN * 128);
                    pa[b] = *reinterpret_cast<const uint32_t *>(plane + row_a * 128 + off);
                    pb[b] = *reinterpret_cast<const uint32_t *>(plane + (row_a + 8) * 128 + off);
                }
                uint32_t ra[8], rb[8];
                planes_to_bytes<Q>(pa, a.w_signed != 0, ra);
                planes_to_bytes<Q>(pb, a.w_signed != 0, rb);
                const uint8_t *rec = rec_base + (size_t)gl * kRec;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt) {
                        const uint2 bf = *reinterpret_cast<const uint2 *>(rec + ((i * MT + mt) * 32 + lane) * 8);
                        mma_u8<XU8>(acc[mt], ra[2 * i], rb[2 * i], ra[2 * i + 1], rb[2 * i + 1], bf.x, bf.y);
                    }
                }
                const int *sums = reinterpret_cast<const int *>(rec + 1024 * MT);
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    const int2 sv = *reinterpret_cast<const int2 *>(sums + 8 * mt + 2 * t);
                    xs[mt][0] += sv.x;
                    xs[mt][1] += sv.y;
                }
                if (grouped) {
                    pending_gi = gi;
                    if ((g_begin + gl + 1) % a.groups_per_scale == 0) {
                        fold(c & 1, gi);
                        pending_gi = -1;
                    }
                }
            }
            // a scale group that continues into the next chunk (or slice) is folded here with the same scale: the
            // fold is linear, and the staged values of this chunk are overwritten two chunks from now
            if (grouped && pending_gi >= 0) {
                fold(c & 1, pending_gi);
                pending_gi = -1;
            }
            __syncwarp();
            if (lane == 0)
                mbar_arrive(&empty[s]);
        }
        __syncwarp();

        // partial result of this slice -> reduce buffer, [token][row] so that the reducer reads rows contiguously
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int row = row_a + 8 * (e >> 1);
                const int tok = 8 * mt + 2 * t + (e & 1);
                int v;
                if (grouped) {
                    v = __float_as_int(facc[mt][e]);
                } else {
                    int z = zoff;
                    const int n = n0 + row;
                    if (a.scale_mode == ABQ_SCALE_CHANNEL && a.w_zero && n < a.N)
                        z += __ldg(a.w_zero + n);
                    v = acc[mt][e] - z * xs[mt][e & 1];
                }
                red[tok * kDecodeBN + row] = v;
            }
        }
    }

    // ---------------- split-K reduction across the cluster, then the fused epilogue
    const uint32_t nranks = cluster_nctarank();
    const uint32_t rank = cluster_ctarank();
    if (nranks > 1)
        cluster_sync_all();
    else
        __syncthreads();

    const int rows_per_rank = kDecodeBN / (int)nranks;
    const int elems = rows_per_rank * 8 * MT;
    const bool grouped = a.scale_mode == ABQ_SCALE_GROUP;
    for (int e = threadIdx.x; e < elems; e += kDecodeThreads) {
        const int row = (int)rank * rows_per_rank + e % rows_per_rank;
        const int tok = e / rows_per_rank;
        const uint32_t local = smem_u32(&red[tok * kDecodeBN + row]);
        int isum = 0;
        float fsum = 0.f;
        for (uint32_t q = 0; q < nranks; ++q) {
            int v;
            if (nranks > 1) {
                asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(v) : "r"(map_to_cta(local, q)) : "memory");
            } else {
                v = red[tok * kDecodeBN + row];
            }
            if (grouped)
                fsum += __int_as_float(v);
            else
                isum += v;
        }
        const int n = n0 + row;
        if (n < a.N && tok < a.M) {
            const size_t o = (size_t)tok * a.N + n;
            if (a.out_dtype == ABQ_OUT_INT32) {
                reinterpret_cast<int *>(a.D)[o] = isum;
            } else {
                __half h;
                if (a.scale_mode == ABQ_SCALE_TENSOR_COMPAT) {
                    h = __hmul(__int2half_rn(isum), ld_half(a.C));
                } else {
                    float v = grouped ? fsum : (float)isum * __half2float(ld_half(a.w_scale + n));
                    if (a.x_scale)
                        v *= __ldg(a.x_scale + tok);
                    h = __float2half_rn(v);
                }
                reinterpret_cast<__half *>(a.D)[o] = h;
            }
        }
    }
    if (nranks > 1)
        cluster_sync_all(); // nobody may exit while a peer still reads its reduce buffer
}

// ------------------------------------------------------------------------------------------- host side

size_t decode_workspace_bytes(int M, int K)
{
    const int MT = M <= 8 ? 1 : 2;
    return (size_t)(K / 128) * decode_record_bytes(MT);
}

template <int Q, int MT, bool XU8>
static cudaError_t launch_variant(const abq_gemm_state *st, const DecodeArgs &args, cudaStream_t stream)
{
    auto kern = decode_kernel<Q, MT, XU8>;
    static thread_local size_t configured = 0; // per instantiation and thread: largest size already opted in
    if (st->shared_mem_size > configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)st->shared_mem_size);
        if (e != cudaSuccess)
            return e;
        configured = st->shared_mem_size;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(st->grid[0], st->grid[1], 1);
    cfg.blockDim = dim3(kDecodeThreads);
    cfg.dynamicSmemBytes = st->shared_mem_size;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int na = 0;
    attr[na].id = cudaLaunchAttributeClusterDimension;
    attr[na].val.clusterDim.x = 1;
    attr[na].val.clusterDim.y = st->cluster;
    attr[na].val.clusterDim.z = 1;
    ++na;
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
    if (MT == 1)
        return xu8 ? launch_variant<Q, 1, true>(st, args, stream) : launch_variant<Q, 1, false>(st, args, stream);
    return xu8 ? launch_variant<Q, 2, true>(st, args, stream) : launch_variant<Q, 2, false>(st, args, stream);
}

abq_status decode_plan(abq_gemm_state *st)
{
    const abq_gemm_params &p = st->p;
    if (p.M > 16)
        return ABQ_ERR_UNSUPPORTED;
    if (p.scale_mode == ABQ_SCALE_GROUP && (p.group_size % 128 != 0))
        return ABQ_ERR_UNSUPPORTED;
    const int MT = p.M <= 8 ? 1 : 2;
    const int Q = p.w_bits;
    const int n_tiles = (p.N + kDecodeBN - 1) / kDecodeBN;
    const int chunks_total = (p.K + kDecodeChunkK - 1) / kDecodeChunkK;
    int sms = 148;
    {
        int dev = 0;
        if (cudaGetDevice(&dev) == cudaSuccess) {
            int v = 0;
            if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && v > 0)
                sms = v;
        }
    }
    // split-K factor: enough CTAs for two per SM, as long as every slice keeps at least one chunk
    int split = 1;
    while (split < 8 && n_tiles * split < 2 * sms && chunks_total >= split * 2)
        split *= 2;
    split = env_int("ABQ_DECODE_SPLITK", split);
    if (split < 1 || split > 8 || (split & (split - 1)) || kDecodeBN % split)
        return ABQ_ERR_INVALID_ARG;
    const int chunks_per_cta = (chunks_total + split - 1) / split;
    const int stage_bytes = Q * kDecodeBN * 128;
    int stages = chunks_per_cta < 4 ? chunks_per_cta : 4;
    while (stages > 1 && stages * stage_bytes > 96 * 1024)
        --stages;
    stages = env_int("ABQ_DECODE_STAGES", stages);
    if (stages < 1 || stages > kMaxStages)
        return ABQ_ERR_INVALID_ARG;
    const int rec_bytes = chunks_per_cta * 8 * decode_record_bytes(MT);
    const size_t smem = 1024 + (size_t)stages * stage_bytes + rec_bytes + (size_t)kDecodeBN * 8 * MT * 4 +
                        (size_t)kConsumerWarps * kScaleStageWords * 4 + (2 * kMaxStages + 1) * 8;
    if (smem > 227 * 1024)
        return ABQ_ERR_UNSUPPORTED;
    if (p.workspace_bytes < decode_workspace_bytes(p.M, p.K) || !p.workspace)
        return ABQ_ERR_WORKSPACE;

    const uint64_t KW = (uint64_t)p.K / 32;
    const uint64_t dims[3] = { KW, (uint64_t)p.N, (uint64_t)Q };
    const uint64_t strides[2] = { KW * 4, KW * 4 * (uint64_t)p.N };
    const uint32_t box[3] = { 32, (uint32_t)kDecodeBN, (uint32_t)Q };
    if (!encode_tmap(st->tmap[0], TMAP_U32, 3, p.W, dims, strides, box, TMAP_SWIZZLE_128B))
        return ABQ_ERR_CUDA;

    st->grid[0] = n_tiles;
    st->grid[1] = split;
    st->grid[2] = 1;
    st->block[0] = kDecodeThreads;
    st->block[1] = st->block[2] = 1;
    st->cluster = split;
    st->shared_mem_size = smem;
    st->tile[0] = chunks_per_cta;
    st->tile[1] = stages;
    st->tile[2] = rec_bytes;
    st->tile[3] = MT;
    return ABQ_OK;
}

cudaError_t decode_launch(const abq_gemm_state *st, cudaStream_t stream)
{
    const abq_gemm_params &p = st->p;
    const int MT = st->tile[3];
    const bool pdl = (p.flags & ABQ_FLAG_PDL) != 0;
    cudaError_t e = xprep_decode(reinterpret_cast<const uint32_t *>(p.X), p.workspace, p.M, p.K, p.x_bits, p.x_signed, MT, pdl, stream);
    if (e != cudaSuccess)
        return e;
    DecodeArgs a;
    a.M = p.M;
    a.N = p.N;
    a.K = p.K;
    a.chunks_per_cta = st->tile[0];
    a.stages = st->tile[1];
    a.rec_smem_bytes = st->tile[2];
    a.records = reinterpret_cast<const uint8_t *>(p.workspace);
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
    case 1: return launch_q<1>(st, a, MT, xu8, stream);
    case 2: return launch_q<2>(st, a, MT, xu8, stream);
    case 3: return launch_q<3>(st, a, MT, xu8, stream);
    case 4: return launch_q<4>(st, a, MT, xu8, stream);
    case 5: return launch_q<5>(st, a, MT, xu8, stream);
    case 6: return launch_q<6>(st, a, MT, xu8, stream);
    case 7: return launch_q<7>(st, a, MT, xu8, stream);
    case 8: return launch_q<8>(st, a, MT, xu8, stream);
    default: return cudaErrorInvalidValue;
    }
}

} // namespace abq
