// Decode route (ABQ_ROUTE_I8_MMA): planner and launch entry.  The kernel lives in gemm_decode_kernel.cuh and is
// instantiated per weight width in gemm_decode_w1.cu .. gemm_decode_w8.cu.
#include "gemm_decode_kernel.cuh"

namespace abq {

struct DecodeLayout {
    int MT, NW, tiles, total_groups, slices, stages_per_slice, ctas_per_slice, split, stages_per_split, ring;
    size_t smem, off_partials, bytes;
};

static int device_sms()
{
    int dev = 0, v = 0;
    if (cudaGetDevice(&dev) == cudaSuccess && cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && v > 0)
        return v;
    return 148;
}

// Workspace (only used when K is split over CTAs): [tile counters][partial slots for kDecodeMaxSlices slices]
void decode_workspace_layout(int M, int N, size_t *off_partials, size_t *total)
{
    const int tiles = (N + 15) / 16;
    const int rows = M < 16 ? M : 16; // taller problems run as launches of 16 rows, one after the other
    *off_partials = ((size_t)tiles * 4 + 255) & ~(size_t)255;
    *total = *off_partials + (size_t)kDecodeMaxSlices * tiles * rows * 16 * 4;
}

size_t decode_workspace_bytes(int M, int N, int K)
{
    (void)K;
    size_t a, total;
    decode_workspace_layout(M, N, &a, &total);
    return total;
}

// Launch shape.  K is split over CTAs only as far as needed for the activation records of a slice to fit beside a
// ring of at least two stages per warp; the tiles are then shared evenly by the CTAs of a slice, and the warps of
// a CTA share a tile `split` ways so that the longest warp (rounds x stages per part) is as short as possible.
static bool make_layout(const abq_gemm_params &p, DecodeLayout *L)
{
    const int Q = p.w_bits;
    const int rows = p.M < 16 ? p.M : 16; // rows per launch
    L->MT = rows <= 8 ? 1 : 2;
    L->tiles = (p.N + 15) / 16;
    L->total_groups = p.K / 128;
    const int total_stages = (L->total_groups + 3) / 4;
    const int sms = device_sms();
    const int stage_bytes = Q * 1024;
    const int rec = decode_record_bytes(L->MT);
    (void)rows;
    const size_t budget = 226 * 1024;
    int t_warps, t_slices, t_ring, t_split; // from the tuning table (0: heuristic); environment variables outrank it
    decode_table_hints(p, &t_warps, &t_slices, &t_ring, &t_split);
    const int forced_slices = env_int("ABQ_DECODE_SLICES", t_slices);
    // 16 warps per CTA when two ring stages per warp fit, else 8 (wide weights); the smallest K split that fits
    int NW = 0, slices = 0, sps = 0, ring = 0;
    size_t fixed = 0;
    for (int nw = env_int("ABQ_DECODE_WARPS", t_warps == 8 || t_warps == 16 ? t_warps : kMaxWarps); nw >= 8 && !NW; nw -= 8) {
        fixed = 1024 + (size_t)nw * 4 * L->MT * 32 * 4 + ((size_t)nw * kMaxRing + 2 * nw) * 8;
        for (int sl = forced_slices > 0 ? forced_slices : 1; sl <= kDecodeMaxSlices && sl <= total_stages; ++sl) {
            const int st = (total_stages + sl - 1) / sl;
            const size_t need = fixed + (size_t)st * 4 * rec;
            const int rg = need < budget ? (int)((budget - need) / ((size_t)nw * stage_bytes)) : 0;
            if (rg >= 2 || (rg >= 1 && nw == 8 && (sl == kDecodeMaxSlices || sl == total_stages)) || (forced_slices > 0 && rg >= 1)) {
                NW = nw;
                slices = sl;
                sps = st;
                ring = rg;
                break;
            }
            if (forced_slices > 0)
                break;
        }
    }
    if (!NW)
        return false;
    slices = (total_stages + sps - 1) / sps; // drop slices that would be empty
    ring = ring > kMaxRing ? kMaxRing : ring;
    ring = env_int("ABQ_DECODE_RING", t_ring > 0 && t_ring <= ring ? t_ring : ring);
    if (ring < 1 || ring > kMaxRing)
        return false;
    int cps = sms / slices;
    cps = cps > L->tiles ? L->tiles : cps;
    cps = cps < 1 ? 1 : cps;
    const int tiles_per_cta = (L->tiles + cps - 1) / cps;
    int best_split = 1;
    long best_cost = -1;
    for (int sp = 1; sp <= NW && sp <= sps; ++sp) {
        const int per_round = NW / sp;
        const long rounds = (tiles_per_cta + per_round - 1) / per_round;
        // in eighths of a stage time: the stages of the longest part, plus per round about one and a half stage times of
        // tile set-up (first scales, output) and, when the tile is shared, of the hand-shake in shared memory
        const long cost = rounds * (((sps + sp - 1) / sp) * 8 + 6 + (sp > 1 ? 6 : 0));
        if (best_cost < 0 || cost < best_cost) {
            best_cost = cost;
            best_split = sp;
        }
    }
    best_split = env_int("ABQ_DECODE_SPLIT", t_split > 0 && t_split <= NW && t_split <= sps ? t_split : best_split);
    if (best_split < 1 || best_split > NW)
        return false;
    L->NW = NW;
    L->slices = slices;
    L->stages_per_slice = sps;
    L->ctas_per_slice = cps;
    L->split = best_split;
    L->stages_per_split = (sps + best_split - 1) / best_split;
    L->ring = ring;
    L->smem = fixed + (size_t)sps * 4 * rec + (size_t)NW * ring * stage_bytes;
    decode_workspace_layout(p.M, p.N, &L->off_partials, &L->bytes);
    return L->smem <= 227 * 1024;
}

abq_status decode_plan(abq_gemm_state *st, bool clear_counters)
{
    const abq_gemm_params &p = st->p;
    // weights already re-laid-out for this route: the stream kernel (widths and modes it does not take read the planes)
    if ((p.flags & ABQ_FLAG_WEIGHTS_PREPARED) && p.w_prepared && stream_supported(p)) {
        const abq_status s = stream_plan(st, clear_counters);
        if (s != ABQ_ERR_UNSUPPORTED)
            return s; // (a shape the stream kernel has no launch for reads the planes after all)
    }
    if (p.scale_mode == ABQ_SCALE_GROUP && (p.group_size % 128 != 0))
        return ABQ_ERR_UNSUPPORTED;
    DecodeLayout L;
    if (!make_layout(p, &L))
        return ABQ_ERR_UNSUPPORTED;
    if (L.slices > 1 && (!p.workspace || p.workspace_bytes < L.bytes))
        return ABQ_ERR_WORKSPACE;
    if (L.slices > 1 && clear_counters) {
        // K split over CTAs: one arrival counter per tile, zero between launches (every launch leaves them zero).
        // Cleared once here and waited for, so that launches on any stream may follow; a memset node per launch would
        // cost several microseconds and break the programmatic chain between consecutive kernels.
        if (cudaMemsetAsync(p.workspace, 0, (size_t)L.tiles * 4, cudaStreamPerThread) != cudaSuccess ||
            cudaStreamSynchronize(cudaStreamPerThread) != cudaSuccess)
            return ABQ_ERR_CUDA;
    }

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
    st->tile[3] = L.split;
    return ABQ_OK;
}

cudaError_t decode_clear_counters(const abq_gemm_state *st, cudaStream_t stream)
{
    if (st->cluster <= 1)
        return cudaSuccess;
    return cudaMemsetAsync(st->p.workspace, 0, (size_t)((st->p.N + 15) / 16) * 4, stream);
}

cudaError_t decode_launch(const abq_gemm_state *st, cudaStream_t stream)
{
    if (stream_planned(st))
        return stream_launch(st, stream);
    const abq_gemm_params &p = st->p;
    const int MT = (p.M < 16 ? p.M : 16) <= 8 ? 1 : 2; // as planned: by the rows of a full launch
    size_t off_partials, total;
    decode_workspace_layout(p.M, p.N, &off_partials, &total);
    uint8_t *ws = reinterpret_cast<uint8_t *>(p.workspace);
    const int tiles = (p.N + 15) / 16;
    DecodeArgs a;
    a.M = p.M;
    a.N = p.N;
    a.K = p.K;
    a.tiles = tiles;
    a.total_groups = p.K / 128;
    a.slices = st->cluster;
    a.stages_per_slice = st->tile[0];
    a.ctas_per_slice = st->tile[2];
    a.split = st->tile[3];
    a.stages_per_split = (a.stages_per_slice + a.split - 1) / a.split;
    a.tiles_q = tiles / a.ctas_per_slice;
    a.tiles_r = tiles % a.ctas_per_slice;
    a.tiles_per_round = (int)st->block[0] / 32 / a.split;
    a.split_magic = 0xffffffffu / (uint32_t)a.split + 1u;
    a.words_magic = 0xffffffffu / (uint32_t)(a.stages_per_slice * 16) + 1u;
    a.ring = st->tile[1];
    a.X = reinterpret_cast<const uint32_t *>(p.X);
    a.x_plane_words = (size_t)p.M * (p.K / 32);
    a.x_qscale = (p.flags & ABQ_FLAG_X_HALF) ? p.x_quant_scale : nullptr;
    a.x_bits = p.x_bits;
    a.x_signed = p.x_signed;
    a.counters = nullptr;
    a.partials = nullptr;
    if (a.slices > 1) {
        // the arrival counters are zero here: planning (or the one-shot call) cleared them, every launch leaves them zero
        a.counters = reinterpret_cast<int *>(ws);
        a.partials = reinterpret_cast<int *>(ws + off_partials);

    }
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
    // M > 16: one launch per 16 rows, in stream order (they share the workspace); the weights of the later launches
    // come out of L2 where they fit
    const size_t out_row_bytes = (size_t)p.N * (p.out_dtype == ABQ_OUT_INT32 ? 4 : 2);
    for (int m0 = 0; m0 < p.M; m0 += 16) {
        a.M = p.M - m0 < 16 ? p.M - m0 : 16;
        a.X = (p.flags & ABQ_FLAG_X_HALF) ? reinterpret_cast<const uint32_t *>(reinterpret_cast<const __half *>(p.X) + (size_t)m0 * p.K)
                                          : reinterpret_cast<const uint32_t *>(p.X) + (size_t)m0 * (p.K / 32);
        a.D = reinterpret_cast<uint8_t *>(p.D) + (size_t)m0 * out_row_bytes;
        a.x_scale = p.x_scale ? p.x_scale + m0 : nullptr;
        a.residual = p.residual ? reinterpret_cast<const __half *>(p.residual) + (size_t)m0 * p.N : nullptr;
        cudaError_t e;
        switch (p.w_bits) {
        case 1: e = decode_launch_w1(st, a, MT, xu8, stream); break;
        case 2: e = decode_launch_w2(st, a, MT, xu8, stream); break;
        case 3: e = decode_launch_w3(st, a, MT, xu8, stream); break;
        case 4: e = decode_launch_w4(st, a, MT, xu8, stream); break;
        case 5: e = decode_launch_w5(st, a, MT, xu8, stream); break;
        case 6: e = decode_launch_w6(st, a, MT, xu8, stream); break;
        case 7: e = decode_launch_w7(st, a, MT, xu8, stream); break;
        case 8: e = decode_launch_w8(st, a, MT, xu8, stream); break;
        default: e = cudaErrorInvalidValue;
        }
        if (e != cudaSuccess)
            return e;
    }
    return cudaSuccess;
}

} // namespace abq
