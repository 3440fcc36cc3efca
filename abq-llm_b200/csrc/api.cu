// C ABI of the library (include/abq_b200.h): validation, route planning, launches.
#include <cuda.h>
#include <cstdlib>
#include <cstring>

#include "abq_kernels.h"

namespace abq {

static thread_local int g_last_cuda_error = 0;

void set_last_cuda_error(cudaError_t e) { g_last_cuda_error = (int)e; }

int env_int(const char *name, int fallback)
{
    const char *v = std::getenv(name);
    if (!v || !*v)
        return fallback;
    return std::atoi(v);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn()
{
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void *sym = nullptr;
        cudaDriverEntryPointQueryResult qres;
        cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres);
        if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess || !sym) {
            set_last_cuda_error(e != cudaSuccess ? e : cudaErrorSymbolNotFound);
            return nullptr;
        }
        fn = reinterpret_cast<EncodeTiledFn>(sym);
    }
    return fn;
}

bool encode_tmap(void *out128, TmapDtype dtype, int rank, const void *base, const uint64_t *dims, const uint64_t *strides_bytes,
                 const uint32_t *box, TmapSwizzle swizzle)
{
    EncodeTiledFn fn = encode_fn();
    if (!fn)
        return false;
    cuuint64_t gdims[5];
    cuuint64_t gstrides[4];
    cuuint32_t gbox[5], estr[5];
    for (int i = 0; i < rank; ++i) {
        gdims[i] = dims[i];
        gbox[i] = box[i];
        estr[i] = 1;
    }
    for (int i = 0; i + 1 < rank; ++i)
        gstrides[i] = strides_bytes[i];
    CUtensorMap tm;
    CUresult r = fn(&tm, dtype == TMAP_U8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_UINT32, (cuuint32_t)rank,
                    const_cast<void *>(base), gdims, gstrides, gbox, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    swizzle == TMAP_SWIZZLE_128B  ? CU_TENSOR_MAP_SWIZZLE_128B
                    : swizzle == TMAP_SWIZZLE_64B ? CU_TENSOR_MAP_SWIZZLE_64B
                                                  : CU_TENSOR_MAP_SWIZZLE_NONE,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_last_cuda_error(cudaErrorInvalidValue);
        return false;
    }
    static_assert(sizeof(CUtensorMap) == 128, "tensor map size");
    std::memcpy(out128, &tm, sizeof(tm));
    return true;
}

static abq_status validate(const abq_gemm_params &p)
{
    if (!p.X || !p.W || !p.D)
        return ABQ_ERR_INVALID_ARG;
    if (p.M <= 0 || p.N <= 0 || p.K < 128 || p.K % 128 != 0) // engine/test_any_mma.cu:99, abq_gemm_wrapper.cu:100
        return ABQ_ERR_INVALID_ARG;
    if (p.x_bits < 1 || p.x_bits > 8 || p.w_bits < 1 || p.w_bits > 8)
        return ABQ_ERR_INVALID_ARG;
    if (p.bias)
        return ABQ_ERR_UNSUPPORTED; // engine/mma_any/aq_bmma_op.h:79
    if (p.out_dtype != ABQ_OUT_INT32 && p.out_dtype != ABQ_OUT_FP16)
        return ABQ_ERR_INVALID_ARG;
    if (p.out_dtype == ABQ_OUT_INT32 && p.scale_mode != ABQ_SCALE_NONE)
        return ABQ_ERR_INVALID_ARG;
    if (p.out_dtype == ABQ_OUT_FP16) {
        switch (p.scale_mode) {
        case ABQ_SCALE_TENSOR_COMPAT:
            if (!p.C)
                return ABQ_ERR_INVALID_ARG;
            break;
        case ABQ_SCALE_CHANNEL:
            if (!p.w_scale)
                return ABQ_ERR_INVALID_ARG;
            break;
        case ABQ_SCALE_GROUP:
            if (!p.w_scale || p.group_size <= 0 || p.K % p.group_size != 0 || p.group_size % 32 != 0)
                return ABQ_ERR_INVALID_ARG;
            break;
        default:
            return ABQ_ERR_INVALID_ARG;
        }
    }
    // the kernels move operands and results in 16-byte pieces: a misaligned pointer would fault on the device
    if ((reinterpret_cast<uintptr_t>(p.X) | reinterpret_cast<uintptr_t>(p.W) | reinterpret_cast<uintptr_t>(p.D)) & 15)
        return ABQ_ERR_INVALID_ARG;
    if (p.residual && (p.out_dtype != ABQ_OUT_FP16 || (reinterpret_cast<uintptr_t>(p.residual) & 1)))
        return ABQ_ERR_INVALID_ARG;
    if (p.flags & ABQ_FLAG_X_HALF) {
        if (!p.x_quant_scale || !p.x_signed)
            return ABQ_ERR_INVALID_ARG;
        if (p.route == ABQ_ROUTE_B1_MMA)
            return ABQ_ERR_UNSUPPORTED; // the 1-bit route multiplies planes
    }
    return ABQ_OK;
}

} // namespace abq

using namespace abq;

extern "C" {

const char *abq_version(void) { return "abq_b200 0.1 sm_100a"; }

const char *abq_status_string(abq_status s)
{
    switch (s) {
    case ABQ_OK: return "ok";
    case ABQ_ERR_INVALID_ARG: return "invalid argument";
    case ABQ_ERR_UNSUPPORTED: return "unsupported request (no kernel for it)";
    case ABQ_ERR_WORKSPACE: return "workspace missing or too small";
    case ABQ_ERR_CUDA: return "CUDA call failed";
    case ABQ_ERR_NOT_INITIALIZED: return "state not initialised";
    case ABQ_ERR_DEVICE_TIMEOUT: return "a bounded device-side wait expired";
    }
    return "unknown status";
}

int abq_last_cuda_error(void) { return g_last_cuda_error; }

size_t abq_gemm_workspace_bytes(int M, int N, int K, int x_bits, int w_bits, int route)
{
    (void)x_bits;
    (void)w_bits;
    size_t need = 0;
    if (route == ABQ_ROUTE_AUTO || route == ABQ_ROUTE_I8_MMA) // AUTO may take this route at any M (per-group scales)
        need = decode_workspace_bytes(M, N, K);
    if (route == ABQ_ROUTE_I8_UMMA || (route == ABQ_ROUTE_AUTO && M > 16)) {
        size_t u = umma_workspace_bytes(M, N, K);
        need = u > need ? u : need;
    }
    return (need + 255) & ~(size_t)255;
}

size_t abq_gemm_prepared_weight_bytes(const abq_gemm_params *params)
{
    if (!params || params->N <= 0 || params->K < 128 || params->K % 128 != 0)
        return 0;
    return stream_prepared_bytes(*params);
}

static abq_status plan_gemm(const abq_gemm_params *params, abq_gemm_state *state, bool clear_counters)
{
    if (!params || !state)
        return ABQ_ERR_INVALID_ARG;
    std::memset(state, 0, sizeof(*state));
    state->p = *params;
    abq_status s = validate(*params);
    if (s != ABQ_OK)
        return s;
    if (params->allreduce) {
        const abq_fused_allreduce &ar = *params->allreduce;
        if (ar.world < 2 || ar.world > 8 || ar.rank < 0 || ar.rank >= ar.world || !ar.counter || ar.rows_cap < params->M)
            return ABQ_ERR_INVALID_ARG;
        for (int r = 0; r < ar.world; ++r)
            if (!ar.recv[r] || !ar.flags[r] || (reinterpret_cast<uintptr_t>(ar.recv[r]) & 15))
                return ABQ_ERR_INVALID_ARG;
        if (params->out_dtype != ABQ_OUT_FP16)
            return ABQ_ERR_INVALID_ARG;
        state->ar = ar; // the copy in the state is what the launch uses (the pointer is dropped once the plan is made)
    }
    int route = params->route;
    if (route == ABQ_ROUTE_AUTO) {
        // up to 16 rows: one launch of the mma.sync route.  17..32 rows: two such launches still beat the tensor-core
        // route, whose weight expansion alone costs more (measured on 12288x4096 and 4096x11008), unless the weight
        // codes are already expanded.  Above: tcgen05.
        const int small = (params->flags & ABQ_FLAG_WEIGHTS_PREPARED) ? 16 : 32;
        route = params->M <= small ? ABQ_ROUTE_I8_MMA : ABQ_ROUTE_I8_UMMA;
    }
    if (params->route == ABQ_ROUTE_AUTO && route == ABQ_ROUTE_I8_UMMA && params->scale_mode == ABQ_SCALE_GROUP) {
        // per-group scales: the tensor-core route drains its accumulator per group where it can (whole K blocks per group,
        // zero points foldable into int8 codes); otherwise the mma.sync route, 16 rows per launch
        s = umma_plan(state);
        if (s == ABQ_ERR_UNSUPPORTED)
            route = ABQ_ROUTE_I8_MMA;
    }
    switch (route) {
    case ABQ_ROUTE_B1_MMA: s = b1_plan(state); break;
    case ABQ_ROUTE_I8_MMA: s = decode_plan(state, clear_counters); break;
    case ABQ_ROUTE_I8_UMMA: s = umma_plan(state); break;
    default: s = ABQ_ERR_INVALID_ARG;
    }
    if (s != ABQ_OK)
        return s;
    if (params->residual && route != ABQ_ROUTE_I8_MMA)
        return ABQ_ERR_UNSUPPORTED; // the residual add lives in the decode kernels' epilogues
    state->route = route;
    state->p.allreduce = nullptr;
    if (state->ar.world > 0 && !(route == ABQ_ROUTE_I8_MMA && stream_planned(state) && state->cluster == 1))
        return ABQ_ERR_UNSUPPORTED; // the fused all-reduce lives in the epilogue of the prepared-weights decode kernel
    state->init_success = 1;
    return ABQ_OK;
}

abq_status abq_gemm_exec(const abq_gemm_state *state, abq_stream_t stream)
{
    if (!state || !state->init_success)
        return ABQ_ERR_NOT_INITIALIZED;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    cudaError_t e;
    switch (state->route) {
    case ABQ_ROUTE_B1_MMA: e = b1_launch(state, st); break;
    case ABQ_ROUTE_I8_MMA: e = decode_launch(state, st); break;
    case ABQ_ROUTE_I8_UMMA: e = umma_launch(state, st); break;
    default: return ABQ_ERR_NOT_INITIALIZED;
    }
    if (e != cudaSuccess) {
        set_last_cuda_error(e);
        return ABQ_ERR_CUDA;
    }
    return ABQ_OK;
}

abq_status abq_gemm_init(const abq_gemm_params *params, abq_gemm_state *state)
{
    return plan_gemm(params, state, true);
}

abq_status abq_gemm_prepare_weights(const abq_gemm_state *state, abq_stream_t stream)
{
    if (!state || !state->init_success)
        return ABQ_ERR_NOT_INITIALIZED;
    if (state->route == ABQ_ROUTE_I8_MMA && !stream_planned(state))
        return ABQ_OK;
    if (state->route != ABQ_ROUTE_I8_UMMA && state->route != ABQ_ROUTE_I8_MMA)
        return ABQ_OK;
    cudaError_t e = state->route == ABQ_ROUTE_I8_MMA ? stream_prepare_weights(state, reinterpret_cast<cudaStream_t>(stream))
                                                     : umma_prepare_weights(state, reinterpret_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) {
        set_last_cuda_error(e);
        return ABQ_ERR_CUDA;
    }
    return ABQ_OK;
}

// Plans of the one-shot entry, kept per host thread: a caller that launches the same GEMM again (a wrapper class called once
// per layer and token step) skips validation, planning and the driver's tensor-map encoding.  A plan depends on nothing but the
// parameter block and the device, so equal bytes mean an equal plan; differing padding bytes only cost a miss.
namespace {
struct CachedPlan {
    abq_gemm_params key;
    int device;
    bool used;
    abq_gemm_state state;
};
constexpr int kPlanCacheEntries = 32;
thread_local CachedPlan g_plan_cache[kPlanCacheEntries];
thread_local int g_plan_cache_next = 0;
} // namespace

abq_status abq_gemm(const abq_gemm_params *params, abq_stream_t stream)
{
    if (!params)
        return ABQ_ERR_INVALID_ARG;
    const abq_gemm_state *plan = nullptr;
    abq_gemm_state fresh;
    int device = -1;
    const bool cacheable = params->allreduce == nullptr && cudaGetDevice(&device) == cudaSuccess; // a pointed-to block may change
    if (cacheable)
        for (int i = 0; i < kPlanCacheEntries && !plan; ++i) {
            const CachedPlan &c = g_plan_cache[i];
            if (c.used && c.device == device && std::memcmp(&c.key, params, sizeof(*params)) == 0)
                plan = &c.state;
        }
    if (!plan) {
        abq_status s = plan_gemm(params, &fresh, false); // one-shot: everything, the counter reset included, goes on the stream
        if (s != ABQ_OK)
            return s;
        plan = &fresh;
        if (cacheable) {
            CachedPlan &c = g_plan_cache[g_plan_cache_next];
            g_plan_cache_next = (g_plan_cache_next + 1) % kPlanCacheEntries;
            c.key = *params;
            c.device = device;
            c.state = fresh;
            c.used = true;
            plan = &c.state;
        }
    }
    if (plan->route == ABQ_ROUTE_I8_MMA) {
        cudaError_t e = decode_clear_counters(plan, reinterpret_cast<cudaStream_t>(stream));
        if (e != cudaSuccess) {
            set_last_cuda_error(e);
            return ABQ_ERR_CUDA;
        }
    }
    return abq_gemm_exec(plan, stream);
}

static abq_status check_pack_args(const void *in, const void *planes, int rows, int K, int bits)
{
    if (!in || !planes || rows <= 0 || K < 128 || K % 128 != 0 || bits < 1 || bits > 8)
        return ABQ_ERR_INVALID_ARG;
    if ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(planes)) & 15) // 16-byte vector loads and stores
        return ABQ_ERR_INVALID_ARG;
    return ABQ_OK;
}

static abq_status wrap(cudaError_t e)
{
    if (e != cudaSuccess) {
        set_last_cuda_error(e);
        return ABQ_ERR_CUDA;
    }
    return ABQ_OK;
}

abq_status abq_pack_int32(const int32_t *in, void *planes, int rows, int K, int bits, abq_stream_t stream)
{
    abq_status s = check_pack_args(in, planes, rows, K, bits);
    if (s != ABQ_OK)
        return s;
    return wrap(pack_int32(in, reinterpret_cast<uint32_t *>(planes), rows, K, bits, reinterpret_cast<cudaStream_t>(stream)));
}

abq_status abq_pack_int4(const void *in, void *planes, int rows, int K, int bits, abq_stream_t stream)
{
    abq_status s = check_pack_args(in, planes, rows, K, bits);
    if (s != ABQ_OK)
        return s;
    if (bits > 4)
        return ABQ_ERR_INVALID_ARG;
    return wrap(pack_int4(in, reinterpret_cast<uint32_t *>(planes), rows, K, bits, reinterpret_cast<cudaStream_t>(stream)));
}

abq_status abq_quantize_pack_half(const void *in_half, const float *scale, void *planes, int rows, int K, int bits, int mode,
                                  abq_stream_t stream)
{
    abq_status s = check_pack_args(in_half, planes, rows, K, bits);
    if (s != ABQ_OK)
        return s;
    if (!scale || (mode != 0 && mode != 1))
        return ABQ_ERR_INVALID_ARG;
    return wrap(quantize_pack_half(reinterpret_cast<const __half *>(in_half), scale, reinterpret_cast<uint32_t *>(planes), rows, K,
                                   bits, mode, reinterpret_cast<cudaStream_t>(stream)));
}

abq_status abq_quantize_weights_half(const void *w_half, int N, int K, int bits, int group_size, int symmetric, void *planes, void *scale_half,
                                     uint8_t *zero, abq_stream_t stream)
{
    abq_status s = check_pack_args(w_half, planes, N, K, bits);
    if (s != ABQ_OK)
        return s;
    if (!scale_half || !zero || group_size < 0 || (group_size > 0 && (group_size % 32 != 0 || K % group_size != 0)) || K > 32768 * 4)
        return ABQ_ERR_INVALID_ARG;
    if (symmetric && bits < 2)
        return ABQ_ERR_INVALID_ARG;
    if (reinterpret_cast<uintptr_t>(scale_half) & 1)
        return ABQ_ERR_INVALID_ARG;
    return wrap(quantize_weights(reinterpret_cast<const __half *>(w_half), reinterpret_cast<uint32_t *>(planes), reinterpret_cast<__half *>(scale_half),
                                 zero, N, K, bits, group_size, symmetric != 0, reinterpret_cast<cudaStream_t>(stream)));
}

abq_status abq_unpack_int8(const void *planes, void *out_i8, int rows, int K, int bits, int is_signed, abq_stream_t stream)
{
    abq_status s = check_pack_args(planes, out_i8, rows, K, bits);
    if (s != ABQ_OK)
        return s;
    return wrap(unpack_i8(reinterpret_cast<const uint32_t *>(planes), out_i8, rows, K, bits, is_signed,
                          reinterpret_cast<cudaStream_t>(stream)));
}

} // extern "C"
