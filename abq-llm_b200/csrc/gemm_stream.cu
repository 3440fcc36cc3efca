// Decode route over prepared weights (stream layout, gemm_stream_kernel.cuh): planner, load-time re-layout and launch
// entry.  The kernel is instantiated per weight width in gemm_stream_w2.cu .. gemm_stream_w8.cu.
#include <dlfcn.h>

#include <cstdio>
#include <cstdlib>
#include <mutex>
#include <string>
#include <vector>

#include "gemm_stream_kernel.cuh"

namespace abq {

namespace {

// What abq_gemm_init decided for this route, kept in the state's route-specific words (tmap[1]).
struct StreamPlan {
    int magic;
    int uw, nw, cu, ring, prefill, slices, units_per_slice, ctas_per_slice, MT, MP, grouped, unit_bytes, max_tiles_per_cta;
    int rows_per_launch; // 16, or 32 (MT == 4) for problems of more than 16 token rows
};
constexpr int kStreamMagic = 0x5354524d;

int device_sms()
{
    int dev = 0, v = 0;
    if (cudaGetDevice(&dev) == cudaSuccess && cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && v > 0)
        return v;
    return 148;
}

bool width_supported(int q) { return q == 2 || q == 3 || q == 4 || q == 8; }

// Launch-shape choices that override the planner's heuristic; 0 = not given.  They come from environment variables
// (ABQ_STREAM_MP / _CU / _RING / _WARPS / _FULL / _CTAS / _SLICES / _PREFILL: tuning runs) or, failing that, from the
// entry of this problem in the tuning table -- the successor of the reference's "time every configuration, keep the best
// per shape" (engine/test/test_mma/test_mma.h:33-46), written by abq-llm_b200/tune.py.
struct StreamHints {
    int mp, cu, ring, warps, full, ctas, slices, prefill;
    int planes; // 1: this problem runs faster on the kernel that reads the planes themselves (no stream plan)
};

struct TuneEntry {
    int w_bits, x_bits, rows_class, N, K, grouped, group_size;
    StreamHints h;
};

int rows_class_of(int M)
{
    return M == 1 ? 1 : M == 2 ? 2 : M <= 4 ? 4 : M <= 8 ? 8 : M <= 16 ? 16 : 32;
}

// Table file: text, one entry per line, '#' starts a comment:
//   w_bits x_bits rows_class N K grouped group_size : mp cu ring warps full ctas slices prefill planes
// Path: ABQ_TUNE_TABLE, else abq_tune_table.txt beside the shared library.  Read once per process.
const std::vector<TuneEntry> &tune_table()
{
    static std::vector<TuneEntry> table;
    static std::once_flag once;
    std::call_once(once, [] {
        std::string path;
        if (const char *e = std::getenv("ABQ_TUNE_TABLE")) {
            path = e;
        } else {
            Dl_info info;
            if (dladdr(reinterpret_cast<const void *>(&rows_class_of), &info) && info.dli_fname) {
                path = info.dli_fname;
                const size_t slash = path.find_last_of('/');
                path = (slash == std::string::npos ? std::string(".") : path.substr(0, slash)) + "/abq_tune_table.txt";
            }
        }
        if (path.empty())
            return;
        FILE *f = std::fopen(path.c_str(), "r");
        if (!f)
            return;
        char line[512];
        while (std::fgets(line, sizeof(line), f)) {
            if (line[0] == '#')
                continue;
            TuneEntry t = {};
            if (std::sscanf(line, "%d %d %d %d %d %d %d : %d %d %d %d %d %d %d %d %d", &t.w_bits, &t.x_bits, &t.rows_class, &t.N, &t.K, &t.grouped,
                            &t.group_size, &t.h.mp, &t.h.cu, &t.h.ring, &t.h.warps, &t.h.full, &t.h.ctas, &t.h.slices, &t.h.prefill, &t.h.planes) == 16)
                table.push_back(t);
        }
        std::fclose(f);
    });
    return table;
}

StreamHints hints_for(const abq_gemm_params &p, int rows)
{
    StreamHints h = {};
    if (!env_int("ABQ_TUNE_IGNORE", 0)) {
        const int grouped = p.scale_mode == ABQ_SCALE_GROUP;
        for (const TuneEntry &t : tune_table()) {
            if (t.w_bits == p.w_bits && t.x_bits == p.x_bits && t.rows_class == rows_class_of(rows) && t.N == p.N && t.K == p.K && t.grouped == grouped &&
                (!grouped || t.group_size == p.group_size)) {
                h = t.h;
                break;
            }
        }
    }
    const struct {
        const char *name;
        int *field;
    } env[] = { { "ABQ_STREAM_MP", &h.mp },     { "ABQ_STREAM_CU", &h.cu },     { "ABQ_STREAM_RING", &h.ring },     { "ABQ_STREAM_WARPS", &h.warps },
                { "ABQ_STREAM_FULL", &h.full }, { "ABQ_STREAM_CTAS", &h.ctas }, { "ABQ_STREAM_SLICES", &h.slices }, { "ABQ_STREAM_PREFILL", &h.prefill },
                { "ABQ_STREAM_PLANES", &h.planes } };
    for (const auto &e : env) {
        const int v = env_int(e.name, -1);
        if (v >= 0)
            *e.field = v;
    }
    return h;
}

// input features per unit: 128, or 64 when the scale groups are an odd multiple of 64 wide
int unit_width_of(const abq_gemm_params &p) { return p.scale_mode == ABQ_SCALE_GROUP && p.group_size % 128 != 0 ? 64 : 128; }

int unit_bytes_of(const abq_gemm_params &p) { return p.w_bits * 2 * unit_width_of(p) + (p.scale_mode == ABQ_SCALE_GROUP ? 64 : 0); }

} // namespace

// The tuning table's launch shape for the kernel that reads the planes (entries with planes = 1 reuse four columns:
// warps, slices, ring, and cu = the number of warps that share a tile along K); zeros where it leaves the heuristic alone.
void decode_table_hints(const abq_gemm_params &p, int *warps, int *slices, int *ring, int *split)
{
    *warps = *slices = *ring = *split = 0;
    if (env_int("ABQ_TUNE_IGNORE", 0))
        return;
    const int grouped = p.scale_mode == ABQ_SCALE_GROUP;
    const int rows = p.M < 16 ? p.M : 16;
    for (const TuneEntry &t : tune_table()) {
        if (t.w_bits == p.w_bits && t.x_bits == p.x_bits && t.rows_class == rows_class_of(rows) && t.N == p.N && t.K == p.K && t.grouped == grouped &&
            (!grouped || t.group_size == p.group_size)) {
            if (t.h.planes > 0) {
                *warps = t.h.warps;
                *slices = t.h.slices;
                *ring = t.h.ring;
                *split = t.h.cu;
            }
            return;
        }
    }
}

bool stream_supported(const abq_gemm_params &p)
{
    if (!width_supported(p.w_bits))
        return false;
    if (!p.x_signed && p.x_bits == 8)
        return false; // unsigned 8-bit activations need the u8 x u8 MMA: the plane kernel has it
    if (p.scale_mode == ABQ_SCALE_GROUP && p.group_size % 64 != 0)
        return false;
    return true;
}

size_t stream_prepared_bytes(const abq_gemm_params &p)
{
    if (!stream_supported(p))
        return 0;
    return (size_t)((p.N + 15) / 16) * (p.K / unit_width_of(p)) * unit_bytes_of(p);
}

// Launch shape.  Preference: a CTA small enough for two to share an SM (so that the next GEMM's CTAs move in and fetch
// their first weights while this one computes), K split over CTAs only when the activation records of the whole K
// range do not fit, chunks of about 4 KB, as deep a ring as the shared memory left over allows.
static bool make_plan_rows(const abq_gemm_params &p, int rows, StreamPlan *P, size_t *smem_bytes)
{
    const bool grouped = p.scale_mode == ABQ_SCALE_GROUP;
    P->magic = kStreamMagic;
    P->grouped = grouped;
    P->MT = rows > 16 ? 4 : rows > 8 ? 2 : 1;
    P->unit_bytes = unit_bytes_of(p);
    P->uw = unit_width_of(p);
    // token rows per column block: the fewest that hold the tokens, but more (fewer units per fold) while a block of
    // 8 / MP units would be too large a chunk for the ring
    const StreamHints H = hints_for(p, rows);
    if (H.planes > 0 && !p.allreduce)
        return false;
    int MP = P->MT >= 2 ? 8 : (rows == 1 ? 1 : rows == 2 ? 2 : rows <= 4 ? 4 : 8);
    while (grouped && MP < 8 && (8 / MP) * P->unit_bytes > 5120)
        MP *= 2;
    if (H.mp > 0 && P->MT == 1)
        MP = H.mp;
    if ((MP != 1 && MP != 2 && MP != 4 && MP != 8) || MP < (rows > 8 ? 8 : rows) || (P->MT >= 2 && MP != 8))
        return false;
    P->MP = MP;
    const int GS = grouped && P->MT == 1 ? 8 / P->MP : 1;
    const int MR = P->MT >= 2 ? 8 * P->MT : P->MP;
    const int units = p.K / P->uw;
    const int tiles = (p.N + 15) / 16;
    const int sms = device_sms();
    const int force_full = H.full;
    const int force_slices = H.slices;
    const int force_warps = H.warps;
    if (force_warps < 0 || force_warps > kStreamMaxWarps || (force_warps & (force_warps - 1)))
        return false; // (a power of two: the kernel shares the chunks out by a shift)
    // Preference: no K split before a K split (its partial sums go through global memory); then eight warps in a CTA that
    // leaves room for a second one on the SM, sixteen in one that fills it, and so on down.
    // A CTA of fewer than eight warps only when no K split makes room for eight.
    for (int pass = 0; pass < 2; ++pass)
    for (int sl = force_slices > 0 ? force_slices : 1; sl <= kDecodeMaxSlices; ++sl) {
        // (two CTAs per SM?, warps) in order of preference
        // (9 to 16 tokens: sixteen warps first -- twice the activation records to expand, twice the MMAs per unit)
        static const int kShapes1[][2] = { { 1, 8 }, { 0, 16 }, { 0, 8 }, { 1, 4 }, { 0, 4 }, { 0, 2 } };
        static const int kShapes2[][2] = { { 0, 16 }, { 1, 8 }, { 0, 8 }, { 1, 4 }, { 0, 4 }, { 0, 2 } };
        static const int kShapes4[][2] = { { 0, 8 }, { 0, 4 } }; // 17..32 tokens: the kernel is built for at most eight warps
        const auto *shapes = P->MT == 4 ? kShapes4 : (P->MT == 2 ? kShapes2 : kShapes1);
        const int n_shapes = P->MT == 4 ? 2 : 6;
        for (int si = 0; si < n_shapes; ++si) {
            const int *shape = shapes[si];
            if ((P->MT == 4 && force_warps > 8) || (force_full == 1 && shape[0]) || (force_full == 2 && !shape[0]) || (!force_warps && (shape[1] >= 8) != (pass == 0)))
                continue; // full: 1 = a CTA that fills the SM, 2 = one that leaves room for a second
            const size_t budget = shape[0] ? 112 * 1024 : 226 * 1024;
            {
                const int nw = force_warps ? force_warps : shape[1];
                int cu0 = H.cu;
                const bool cu_forced = cu0 > 0;
                if (!cu_forced) {
                    cu0 = (4608 / P->unit_bytes) / GS * GS;
                    cu0 = cu0 < GS ? GS : cu0;
                    cu0 = cu0 > 8 ? 8 : cu0;
                }
                if (cu0 % GS != 0)
                    return false;
                // smaller chunks before fewer warps or a K split: the ring of a shape that does not fit is halved first
                for (int cu = cu0; cu >= GS && cu >= (cu_forced ? cu0 : 2) && (cu == cu0 || cu * P->unit_bytes >= 2048); cu = (cu / 2) / GS * GS) {
                int ups = (units + sl - 1) / sl;
                ups = (ups + cu - 1) / cu * cu;
                const int slices = (units + ups - 1) / ups; // drop slices that would be empty
                int cps = (H.ctas > 0 ? H.ctas : sms) / slices;
                cps = cps > tiles ? tiles : cps;
                cps = cps < 1 ? 1 : cps;
                const int max_T = (tiles + cps - 1) / cps;
                const StreamSmem L0 = stream_smem_layout(nw, 0, cu, P->unit_bytes, ups, MR, max_T, P->MT, P->uw);
                if (L0.total < budget && max_T <= 64 && (long long)tiles * (cps + 1) < (1LL << 31)) { // (the kernel keeps a 64-entry table of its tiles)
                    int ring = (int)((budget - L0.total) / ((size_t)nw * cu * P->unit_bytes));
                    ring = ring > kStreamMaxRing ? kStreamMaxRing : ring;
                    const int forced = H.ring;
                    if (forced > 0 && forced <= ring)
                        ring = forced;
                    if (ring >= 2) {
                        P->nw = nw;
                        P->cu = cu;
                        P->ring = ring;
                        P->prefill = H.prefill > 0 ? (H.prefill > ring ? ring : H.prefill) : ring;
                        P->slices = slices;
                        P->units_per_slice = ups;
                        P->ctas_per_slice = cps;
                        P->max_tiles_per_cta = max_T;
                        *smem_bytes = stream_smem_layout(nw, ring, cu, P->unit_bytes, ups, MR, max_T, P->MT, P->uw).total;
                        return true;
                    }
                }
                if (cu == GS)
                    break;
                }
            }
        }
        if (force_slices > 0)
            break;
    }
    return false;
}

// More than 16 token rows: launches of 16 rows.  Launches of 32 rows (the weights are then read once per 32 rows) exist
// and are tested, but are opt-in (ABQ_STREAM_ROWS32=1): every CTA expands the activation records of all 32 rows, and with
// eight warps and one CTA per SM that costs more than the second read of the weights saves (LLaMA-7B W4A4 linear stack at
// batch 32: 5.43 ms per step against 4.23 ms with two 16-row launches per GEMM).
static bool make_plan(const abq_gemm_params &p, StreamPlan *P, size_t *smem_bytes)
{
    if (p.M > 16 && env_int("ABQ_STREAM_ROWS32", 0) != 0 && make_plan_rows(p, p.M < 32 ? p.M : 32, P, smem_bytes)) {
        // a K split parks 32-row partial tiles in the workspace, which callers size for 16-row launches: take it only if they fit
        size_t off_partials, total;
        decode_workspace_layout(p.M, p.N, &off_partials, &total);
        const size_t need = off_partials + (size_t)P->slices * ((p.N + 15) / 16) * 32 * 16 * 4;
        if (P->slices == 1 || (p.workspace && p.workspace_bytes >= need)) {
            P->rows_per_launch = 32;
            return true;
        }
    }
    P->rows_per_launch = 16;
    return make_plan_rows(p, p.M < 16 ? p.M : 16, P, smem_bytes);
}

abq_status stream_plan(abq_gemm_state *st, bool clear_counters)
{
    const abq_gemm_params &p = st->p;
    if (!stream_supported(p) || !p.w_prepared)
        return ABQ_ERR_UNSUPPORTED;
    if (reinterpret_cast<uintptr_t>(p.w_prepared) & 15)
        return ABQ_ERR_INVALID_ARG;
    StreamPlan P;
    size_t smem = 0;
    if (!make_plan(p, &P, &smem))
        return ABQ_ERR_UNSUPPORTED;
    if (P.slices > 1) {
        if (!p.workspace || p.workspace_bytes < decode_workspace_bytes(p.M, p.N, p.K))
            return ABQ_ERR_WORKSPACE;
        if (clear_counters) { // as the plane kernel: cleared once here, every launch leaves them zero
            if (cudaMemsetAsync(p.workspace, 0, (size_t)((p.N + 15) / 16) * 4, cudaStreamPerThread) != cudaSuccess ||
                cudaStreamSynchronize(cudaStreamPerThread) != cudaSuccess)
                return ABQ_ERR_CUDA;
        }
    }
    static_assert(sizeof(StreamPlan) <= sizeof(st->tmap[1]), "plan words");
    std::memcpy(st->tmap[1], &P, sizeof(P));
    st->grid[0] = P.slices * P.ctas_per_slice;
    st->grid[1] = st->grid[2] = 1;
    st->block[0] = P.nw * 32;
    st->block[1] = st->block[2] = 1;
    st->cluster = P.slices;
    st->shared_mem_size = smem;
    st->tile[0] = P.units_per_slice;
    st->tile[1] = P.ring;
    st->tile[2] = P.ctas_per_slice;
    st->tile[3] = P.cu;
    return ABQ_OK;
}

bool stream_planned(const abq_gemm_state *st)
{
    StreamPlan P;
    std::memcpy(&P, st->tmap[1], sizeof(P));
    return st->route == ABQ_ROUTE_I8_MMA && P.magic == kStreamMagic;
}

cudaError_t stream_prepare_weights(const abq_gemm_state *st, cudaStream_t stream)
{
    const abq_gemm_params &p = st->p;
    const int grouped = p.scale_mode == ABQ_SCALE_GROUP;
    const int uw = unit_width_of(p);
    const int gps = grouped ? p.group_size / uw : 1, sg = grouped ? p.K / p.group_size : 1;
    const uint32_t *planes = reinterpret_cast<const uint32_t *>(p.W);
    const __half *ws = reinterpret_cast<const __half *>(p.w_scale);
    uint8_t *out = reinterpret_cast<uint8_t *>(p.w_prepared);
    switch (p.w_bits) {
    case 2: return stream_prepare_w2(planes, ws, p.w_zero, out, p.N, p.K, p.w_signed, grouped, uw, gps, sg, stream);
    case 3: return stream_prepare_w3(planes, ws, p.w_zero, out, p.N, p.K, p.w_signed, grouped, uw, gps, sg, stream);
    case 4: return stream_prepare_w4(planes, ws, p.w_zero, out, p.N, p.K, p.w_signed, grouped, uw, gps, sg, stream);
    case 8: return stream_prepare_w8(planes, ws, p.w_zero, out, p.N, p.K, p.w_signed, grouped, uw, gps, sg, stream);
    }
    return cudaErrorInvalidValue;
}

cudaError_t stream_launch(const abq_gemm_state *st, cudaStream_t stream)
{
    const abq_gemm_params &p = st->p;
    StreamPlan P;
    std::memcpy(&P, st->tmap[1], sizeof(P));
    StreamArgs a;
    a.N = p.N;
    a.K = p.K;
    a.tiles = (p.N + 15) / 16;
    a.uw = P.uw;
    a.units = p.K / P.uw;
    a.unit_bytes = P.unit_bytes;
    a.slices = P.slices;
    a.units_per_slice = P.units_per_slice;
    a.ctas_per_slice = P.ctas_per_slice;
    a.cu = P.cu;
    a.ring = P.ring;
    a.prefill = P.prefill;
    a.nw = P.nw;
    a.nw_shift = 0;
    while ((1 << a.nw_shift) < P.nw)
        ++a.nw_shift;
    a.tiles_q = a.tiles / P.ctas_per_slice;
    a.tiles_r = a.tiles % P.ctas_per_slice;
    a.max_tiles = (a.tiles + P.ctas_per_slice - 1) / P.ctas_per_slice;
    a.cpt_full = (P.units_per_slice + P.cu - 1) / P.cu;
    a.rec_magic = 0xffffffffu / (uint32_t)(P.units_per_slice * (P.uw / 32)) + 1u;
    a.cpt_magic = 0xffffffffu / (uint32_t)a.cpt_full + 1u;
    a.Wp = reinterpret_cast<const uint8_t *>(p.w_prepared);
    a.x_plane_words = (size_t)p.M * (p.K / 32);
    a.x_qscale = (p.flags & ABQ_FLAG_X_HALF) ? p.x_quant_scale : nullptr;
    a.x_bits = p.x_bits;
    a.x_signed = p.x_signed;
    a.counters = nullptr;
    a.partials = nullptr;
    if (P.slices > 1) {
        size_t off_partials, total;
        decode_workspace_layout(p.M, p.N, &off_partials, &total);
        a.counters = reinterpret_cast<int *>(p.workspace);
        a.partials = reinterpret_cast<int *>(reinterpret_cast<uint8_t *>(p.workspace) + off_partials);
    }
    a.w_scale = reinterpret_cast<const __half *>(p.w_scale);
    a.w_zero = p.w_zero;
    a.C = reinterpret_cast<const __half *>(p.C);
    a.out_dtype = p.out_dtype;
    a.scale_mode = p.scale_mode;
    a.w_signed = p.w_signed;
    a.status = p.status_word;
    a.ar.world = st->ar.world;
    a.ar.rank = st->ar.rank;
    a.ar.rows_cap = st->ar.rows_cap;
    a.ar.counter = st->ar.counter;
    for (int r = 0; r < 8; ++r) {
        a.ar.recv[r] = reinterpret_cast<__half *>(st->ar.recv[r]);
        a.ar.flags[r] = st->ar.flags[r];
    }
    const size_t out_row_bytes = (size_t)p.N * (p.out_dtype == ABQ_OUT_INT32 ? 4 : 2);
    const int step = P.rows_per_launch;
    for (int m0 = 0; m0 < p.M; m0 += step) { // taller problems: 16 or 32 rows per launch, in stream order (they share the workspace)
        a.M = p.M - m0 < step ? p.M - m0 : step;
        a.per_tile_magic = 0xffffffffu / (uint32_t)(16 * a.M) + 1u;
        a.X = (p.flags & ABQ_FLAG_X_HALF) ? reinterpret_cast<const uint32_t *>(reinterpret_cast<const __half *>(p.X) + (size_t)m0 * p.K)
                                          : reinterpret_cast<const uint32_t *>(p.X) + (size_t)m0 * (p.K / 32);
        a.D = reinterpret_cast<uint8_t *>(p.D) + (size_t)m0 * out_row_bytes;
        a.x_scale = p.x_scale ? p.x_scale + m0 : nullptr;
        a.residual = p.residual ? reinterpret_cast<const __half *>(p.residual) + (size_t)m0 * p.N : nullptr;
        a.ar.row0 = m0;
        cudaError_t e;
        switch (p.w_bits) {
        case 2: e = stream_launch_w2(st, a, P.MT, P.MP, P.grouped != 0, stream); break;
        case 3: e = stream_launch_w3(st, a, P.MT, P.MP, P.grouped != 0, stream); break;
        case 4: e = stream_launch_w4(st, a, P.MT, P.MP, P.grouped != 0, stream); break;
        case 8: e = stream_launch_w8(st, a, P.MT, P.MP, P.grouped != 0, stream); break;
        default: e = cudaErrorInvalidValue;
        }
        if (e != cudaSuccess)
            return e;
    }
    return cudaSuccess;
}

} // namespace abq
