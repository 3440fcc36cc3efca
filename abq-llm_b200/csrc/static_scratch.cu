// abq_gemm_static_scratch: the GEMM entry point for callers that can neither pass nor allocate scratch memory.
//
// The plane-to-int8 route needs scratch beyond its inputs and outputs (the expanded 8-bit operands and the
// token sums, see gemm_umma.cu).  abq_gemm takes that scratch from the caller.  Some callers cannot provide it:
// the FasterTransformer linear-layer call sites hand the wrapper a workspace sized for the activation planes
// only (x_bits * tokens * K / 8 bytes, allocated by layer code that a drop-in kernel library does not own), and
// inside a layer's forward pass a cudaMalloc is not an option either: it synchronises the device, breaks
// stream-ordered execution, and is forbidden outright while the stream is being captured into a CUDA graph.
// For them this file keeps one fixed scratch array in device memory and this entry point runs the ordinary GEMM on
// top of it.  The array belongs to the library's device code: a GPU holds it from the moment the CUDA runtime loads
// that code on it (with lazy module loading that is the first call below on that GPU) until the process exits.  Nothing here
// (nor anything it calls) calls cudaMalloc, cudaFree or an allocating library routine.
#include <cuda_runtime.h>

#include "abq_kernels.h"

namespace abq {

// The scratch itself.  In host code this name is only a handle for the runtime, not a device address: the
// address a kernel can use comes from cudaGetSymbolAddress, once per device, with that device current.
static __device__ __align__(256) unsigned char g_static_scratch[ABQ_STATIC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
static void *g_scratch_ptr[kMaxDevices] = {};

static cudaError_t static_scratch_address(void **out)
{
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess)
        return e;
    if (dev < 0 || dev >= kMaxDevices)
        return cudaErrorInvalidDevice;
    if (!g_scratch_ptr[dev]) {
        void *p = nullptr;
        e = cudaGetSymbolAddress(&p, g_static_scratch);
        if (e != cudaSuccess)
            return e;
        g_scratch_ptr[dev] = p;
    }
    *out = g_scratch_ptr[dev];
    return cudaSuccess;
}

} // namespace abq

extern "C" abq_status abq_gemm_static_scratch(const abq_gemm_params *params, abq_stream_t stream)
{
    if (!params)
        return ABQ_ERR_INVALID_ARG;
    // "Prepared" weights of the tensor-core route are an expansion that an earlier call left in the plan's own workspace.
    // On the shared array the last call may have been any other GEMM, so whatever sits there is not this problem's
    // weights: refuse.  The decode route keeps its prepared copy in the caller's own buffer (w_prepared) and uses the
    // workspace for split-K partial sums only, so that combination, asked for by name, is served.
    if ((params->flags & ABQ_FLAG_WEIGHTS_PREPARED) && !(params->route == ABQ_ROUTE_I8_MMA && params->w_prepared))
        return ABQ_ERR_INVALID_ARG;
    const size_t need = abq_gemm_workspace_bytes(params->M, params->N, params->K, params->x_bits, params->w_bits, params->route);
    if (need > (size_t)ABQ_STATIC_SCRATCH_BYTES)
        return ABQ_ERR_WORKSPACE; // the problem needs more scratch than the built-in array holds: use abq_gemm with a workspace
    void *scratch = nullptr;
    cudaError_t e = abq::static_scratch_address(&scratch);
    if (e != cudaSuccess) {
        abq::set_last_cuda_error(e);
        return ABQ_ERR_CUDA;
    }
    abq_gemm_params p = *params;
    p.workspace = scratch;
    p.workspace_bytes = (size_t)ABQ_STATIC_SCRATCH_BYTES;
    return abq_gemm(&p, stream);
}
