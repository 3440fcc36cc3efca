// abq_compat.hpp -- the reference's C++ launch interface re-created over the C ABI (abq_b200.h).
//
// Purpose: source that was written against the reference engine keeps compiling when it is pointed at this
// library instead.  Every name below exists in the reference with the same spelling and argument meaning; each
// comment cites where (paths inside the reference repository).  The bodies only fill an abq_gemm_params and call
// the C ABI; tile-shape template arguments and per-configuration function names are accepted and ignored (the
// library plans the tile itself).  Header-only; needs <cuda_runtime.h> and <cuda_fp16.h> like the reference.
//
// Differences a caller can observe:
//   * the planned kernels need caller-owned scratch for M > 16 (see abq_gemm_workspace_bytes); the reference
//     signatures have no place for it, so these shims use abq_gemm_static_scratch (built-in 16 MiB array) unless a
//     workspace was installed with abq_compat::set_workspace();
//   * failures are reported (initSuccess = false / cudaErrorUnknown / a message on stderr), never ignored.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdio>
#include <map>

#include "abq_b200.h"

namespace abq_compat {

struct Workspace {
    void *ptr = nullptr;
    size_t bytes = 0;
};
inline Workspace &workspace()
{
    static thread_local Workspace w;
    return w;
}
// Optional: scratch for GEMMs launched through the shims below (per host thread).
inline void set_workspace(void *device_ptr, size_t bytes)
{
    workspace().ptr = device_ptr;
    workspace().bytes = bytes;
}

// abq_gemm_static_scratch, and for problems whose planned route needs more scratch than the built-in array holds
// (e.g. 128 x 4096 x 4096 on the tensor-core route: 17 MB of expanded operands) the same call on the route that needs
// next to none (16 rows per launch, reading the planes directly): slower, but the reference's signatures leave no way
// to ask the caller for memory.
inline abq_status static_scratch(const abq_gemm_params &p, cudaStream_t stream)
{
    abq_status s = abq_gemm_static_scratch(&p, stream);
    if (s == ABQ_ERR_WORKSPACE && p.route == ABQ_ROUTE_AUTO) {
        abq_gemm_params q = p;
        q.route = ABQ_ROUTE_I8_MMA;
        s = abq_gemm_static_scratch(&q, stream);
    }
    return s;
}

inline abq_status run(abq_gemm_params &p, cudaStream_t stream)
{
    const Workspace &w = workspace();
    if (w.ptr) {
        p.workspace = w.ptr;
        p.workspace_bytes = w.bytes;
        return abq_gemm(&p, stream);
    }
    return static_scratch(p, stream);
}

} // namespace abq_compat

// ---- engine/common/pack.h:20-24 --------------------------------------------------------------------------------
inline cudaError_t launch_pack(const int *in_data, int *pack_data, int m, int k, int BIT, cudaStream_t stream = 0)
{
    return abq_pack_int32(in_data, pack_data, m, k, BIT, stream) == ABQ_OK ? cudaSuccess : cudaErrorUnknown;
}
inline cudaError_t launch_pack4(const int *in_data, int *pack_data, int m, int k, int BIT, cudaStream_t stream = 0)
{
    return abq_pack_int4(in_data, pack_data, m, k, BIT, stream) == ABQ_OK ? cudaSuccess : cudaErrorUnknown;
}

// ---- engine/common/base.h:36-58: compile-time tags, kept so that template argument lists still parse ---------------
template <int M_, int N_, int K_>
struct ShapeBase {
    static constexpr int M = M_, N = N_, K = K_;
};
template <int X_BITS_, int W_BITS_, bool SIGNED_>
struct QuantType {
    static constexpr int X_BITS = X_BITS_, W_BITS = W_BITS_;
    static constexpr bool SIGNED = SIGNED_;
};

// ---- engine/mma_any/aq_bmma_op.h:19-32 (and the identical AqBWMMAOpState, aq_wmma_op.h) ------------------------------
struct AqBMMAOpState {
    size_t shared_mem_size = 0;
    dim3 gridDim, blockDim;
    bool initSuccess = false;
    struct Argument_t {
        int M, N, K;
        int *X;
        int *W;
        half *C;
        int *D;
        bool bias = false;
    } args;
    // extension: the quantisation the state was initialised for, and the plan
    int x_bits = 0, w_bits = 0;
    bool quant_signed = false;
    abq_gemm_state plan;
};
typedef AqBMMAOpState AqBWMMAOpState;

// ---- engine/mma_any/aq_bmma_op.h:141-164: pure-function Init / Exec pair -------------------------------------------
// The reference instantiates one pair per (QuantType, tile shapes, stages); here the tile arguments are ignored.
template <typename QuantT, typename ThreadBlockShape = void, typename WarpShape = void, typename MmaShape = void, int NStage = 0>
AqBMMAOpState AqBMMAInitFn(int *X, int *W, int M, int N, int K, int *D, half *C, bool bias)
{
    AqBMMAOpState st;
    st.args.M = M;
    st.args.N = N;
    st.args.K = K;
    st.args.X = X;
    st.args.W = W;
    st.args.C = C;
    st.args.D = D;
    st.args.bias = bias;
    st.x_bits = QuantT::X_BITS;
    st.w_bits = QuantT::W_BITS;
    st.quant_signed = QuantT::SIGNED;
    abq_gemm_params p = {};
    p.M = M;
    p.N = N;
    p.K = K;
    p.X = X;
    p.W = W;
    p.C = C;
    p.D = D;
    p.bias = bias;
    p.x_bits = QuantT::X_BITS;
    p.w_bits = QuantT::W_BITS;
    p.x_signed = p.w_signed = QuantT::SIGNED;
    p.out_dtype = ABQ_OUT_INT32; // the engine writes raw int32 (aq_bmma_kernel.h:571-575)
    // With an installed workspace the launch is planned once here and Exec only launches; without one Exec goes
    // through abq_gemm_static_scratch, which plans per call.
    const abq_compat::Workspace &w = abq_compat::workspace();
    abq_status s = ABQ_OK;
    st.plan = abq_gemm_state();
    if (w.ptr) {
        p.workspace = w.ptr;
        p.workspace_bytes = w.bytes;
        s = abq_gemm_init(&p, &st.plan);
    } else if (K < 128 || K % 128 != 0 || bias) {
        s = bias ? ABQ_ERR_UNSUPPORTED : ABQ_ERR_INVALID_ARG; // what abq_gemm_init would answer
    }
    st.plan.p = p;
    st.initSuccess = s == ABQ_OK;
    if (!st.initSuccess)
        std::fprintf(stderr, "AqBMMAInitFn: %s\n", abq_status_string(s));
    st.gridDim = dim3(st.plan.grid[0] ? st.plan.grid[0] : 1, st.plan.grid[1] ? st.plan.grid[1] : 1, 1);
    st.blockDim = dim3(st.plan.block[0] ? st.plan.block[0] : 1, 1, 1);
    st.shared_mem_size = st.plan.shared_mem_size;
    return st;
}

template <typename QuantT, typename ThreadBlockShape = void, typename WarpShape = void, typename MmaShape = void, int NStage = 0>
void AqBMMAExecFn(AqBMMAOpState &state, cudaStream_t stream = NULL)
{
    abq_status s;
    if (!state.initSuccess)
        s = ABQ_ERR_NOT_INITIALIZED;
    else if (state.plan.init_success)
        s = abq_gemm_exec(&state.plan, stream);
    else
        s = abq_compat::static_scratch(state.plan.p, stream);
    if (s != ABQ_OK)
        std::fprintf(stderr, "AqBMMAExecFn: %s\n", abq_status_string(s));
}

typedef AqBMMAOpState (*AqBMMAInitFn_t)(int *, int *, int, int, int, int *, half *, bool);
typedef void (*AqBMMAExecFn_t)(AqBMMAOpState &, cudaStream_t);
typedef AqBMMAInitFn_t AqBWMMAInitFn_t;
typedef AqBMMAExecFn_t AqBWMMAExecFn_t;

// engine/common/base.h:144-166: the reference names one global function-pointer pair per configuration, e.g.
// AqBMMA_8x2xtrue_1x48x512_8x24x128_8x8x128_4_InitFn.  ABQ_COMPAT_DEFINE_CONFIG re-creates such a pair; the tile
// part of the name is whatever the caller's code spells.
#define ABQ_COMPAT_DEFINE_CONFIG(NAME, X_BITS, W_BITS, SIGNED)                                                        \
    static AqBMMAInitFn_t NAME##_InitFn = &AqBMMAInitFn<QuantType<X_BITS, W_BITS, SIGNED>>;                            \
    static AqBMMAExecFn_t NAME##_ExecFn = &AqBMMAExecFn<QuantType<X_BITS, W_BITS, SIGNED>>;

// ---- engine/wmma_any/wmma_any.h:18-38 -----------------------------------------------------------------------------
struct AnyQuantParams {
    const int *X;
    const int *W;
    const half *C;
    int *D;
    bool bias = false;
    const int M;
    const int N;
    const int K;
};

template <typename QuantT, typename ThreadBlockShape = void, typename WarpShape = void, typename MmaShape = void, int kThreadBlockStage = 0>
cudaError_t launchWmmaAnyKernel(const AnyQuantParams &params, const cudaStream_t &stream)
{
    abq_gemm_params p = {};
    p.M = params.M;
    p.N = params.N;
    p.K = params.K;
    p.X = params.X;
    p.W = params.W;
    p.C = params.C;
    p.D = params.D;
    p.bias = params.bias;
    p.x_bits = QuantT::X_BITS;
    p.w_bits = QuantT::W_BITS;
    p.x_signed = p.w_signed = QuantT::SIGNED;
    p.out_dtype = ABQ_OUT_INT32;
    return abq_compat::run(p, stream) == ABQ_OK ? cudaSuccess : cudaErrorUnknown;
}

// ---- fastertransformer/src/fastertransformer/kernels/abqgemm/abq_gemm_wrapper.h:6-32 ------------------------------------
// Same class name and method signatures.  gemm() quantises + packs A into the caller's workspace exactly as the
// reference does (int(half(x) * half(scale)), abq_gemm_wrapper.cu:29-54), then multiplies by the pre-packed weight
// planes and writes D = half(acc) * half(scale_out) (the float is read as fp16, abq_gemm_wrapper.cu:125-126).
// Any width 1..8 is accepted (the reference: W2A8 only); the workspace size is checked; errors are printed.
class ABQGEMMWrapper {
private:
    int x_bits_;
    int w_bits_;
    bool signed_;
    std::map<const int *, void *> prepared_; // weight planes -> their prepared copy (extension, see prepare_weights)

public:
    ABQGEMMWrapper(int X_BITS, int W_BITS, bool SIGNED): x_bits_(X_BITS), w_bits_(W_BITS), signed_(SIGNED) {}
    ~ABQGEMMWrapper() {}

    void pack(const int *in_data, int *packed_data, int M, int K, int BIT, cudaStream_t stream)
    {
        report(abq_pack_int32(in_data, packed_data, M, K, BIT, stream), "pack");
    }
    void pack(const half *in_data, const float *scale, int *packed_data, int M, int K, int BIT, cudaStream_t stream)
    {
        report(abq_quantize_pack_half(in_data, scale, packed_data, M, K, BIT, 0, stream), "pack");
    }
    // Extension (no counterpart in the reference): bytes of, and the one-time set-up of, the prepared copy of a weight for
    // decode-shape calls.  Call once per weight where the planes are loaded (LlamaDecoderLayerWeight::loadModel), with a
    // device buffer of prepared_weight_bytes(N, K) bytes that lives as long as the planes; gemm() calls with these planes
    // and up to 32 tokens then read the prepared copy.  Waits for the re-ordering to finish.
    size_t prepared_weight_bytes(int N, int K) const
    {
        abq_gemm_params p = {};
        p.M = 1;
        p.N = N;
        p.K = K;
        p.x_bits = x_bits_;
        p.w_bits = w_bits_;
        p.x_signed = p.w_signed = signed_;
        p.out_dtype = ABQ_OUT_FP16;
        p.scale_mode = ABQ_SCALE_TENSOR_COMPAT;
        return abq_gemm_prepared_weight_bytes(&p);
    }
    bool prepare_weights(const int *B, int N, int K, void *prepared, cudaStream_t stream)
    {
        abq_gemm_params p = {};
        p.M = 1;
        p.N = N;
        p.K = K;
        p.X = B; // (planning needs a non-null, aligned pointer; the activations are not touched here)
        p.W = B;
        p.C = B;
        p.D = prepared;
        p.x_bits = x_bits_;
        p.w_bits = w_bits_;
        p.x_signed = p.w_signed = signed_;
        p.out_dtype = ABQ_OUT_FP16;
        p.scale_mode = ABQ_SCALE_TENSOR_COMPAT;
        p.route = ABQ_ROUTE_I8_MMA;
        p.flags = ABQ_FLAG_WEIGHTS_PREPARED;
        p.w_prepared = prepared;
        abq_gemm_state st;
        abq_status s = abq_gemm_init(&p, &st);
        if (s == ABQ_OK)
            s = abq_gemm_prepare_weights(&st, stream);
        if (s != ABQ_OK || cudaStreamSynchronize(stream) != cudaSuccess) {
            report(s == ABQ_OK ? ABQ_ERR_CUDA : s, "prepare_weights");
            return false;
        }
        prepared_[B] = prepared;
        return true;
    }

    void gemm(const int M, const int N, const int K, const half *A, const int *B, const half *C, half *D, const float *scale,
              const float *scale_inter, const float *scale_out, bool bias, char *abq_gemm_workspace, size_t abq_gemm_ws_bytes,
              cudaStream_t stream)
    {
        (void)C;
        (void)scale_inter; // ignored by the reference as well
        if (K < 128 || K % 128 != 0) {
            std::printf("[ABQ][Error] unsupport K = %d\n", K);
            return;
        }
        const size_t plane_bytes = ((size_t)x_bits_ * M * (K / 32) * 4 + 255) & ~(size_t)255;
        if (abq_gemm_ws_bytes < (size_t)x_bits_ * M * (K / 32) * 4) {
            std::printf("[ABQ][Error] workspace of %zu bytes cannot hold the activation planes\n", abq_gemm_ws_bytes);
            return;
        }
        // signed configurations: the GEMM call quantises the fp16 activations itself (same codes as pack, one launch
        // less, no planes); unsigned ones go through the planes as the reference does
        const bool fused = signed_;
        if (!fused)
            pack(A, scale, reinterpret_cast<int *>(abq_gemm_workspace), M, K, x_bits_, stream);
        abq_gemm_params p = {};
        p.M = M;
        p.N = N;
        p.K = K;
        p.X = fused ? static_cast<const void *>(A) : static_cast<const void *>(abq_gemm_workspace);
        p.flags = fused ? ABQ_FLAG_X_HALF : 0;
        p.x_quant_scale = scale;
        p.W = B;
        p.C = scale_out;
        p.D = D;
        p.bias = bias;
        p.x_bits = x_bits_;
        p.w_bits = w_bits_;
        p.x_signed = p.w_signed = signed_;
        p.out_dtype = ABQ_OUT_FP16;
        p.scale_mode = ABQ_SCALE_TENSOR_COMPAT;
        const auto prep = prepared_.find(B);
        if (prep != prepared_.end() && M <= 32) { // a prepared copy of these planes exists: the decode kernel that reads it
            p.w_prepared = prep->second;
            p.flags |= ABQ_FLAG_WEIGHTS_PREPARED;
            p.route = ABQ_ROUTE_I8_MMA;
        }
        const size_t need = abq_gemm_workspace_bytes(M, N, K, x_bits_, w_bits_, p.route);
        abq_status s;
        const size_t used = fused ? 0 : plane_bytes; // the fused call leaves the whole workspace to the GEMM
        if (abq_gemm_ws_bytes >= used + need) { // a caller that sized the workspace with room for the scratch
            p.workspace = abq_gemm_workspace + used;
            p.workspace_bytes = abq_gemm_ws_bytes - used;
            s = abq_gemm(&p, stream);
        } else { // the reference's layers size it for the planes only
            s = abq_compat::static_scratch(p, stream);
        }
        report(s, "gemm");
    }

private:
    static void report(abq_status s, const char *what)
    {
        if (s != ABQ_OK)
            std::printf("[ABQ][Error] %s: %s\n", what, abq_status_string(s));
    }
};
