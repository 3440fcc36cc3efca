// Host-callable launchers of the kernels in this directory and the layout constants they share.
#pragma once
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <stdint.h>

#include "../../include/abq_b200.h"

namespace abq {

// ---- pack.cu
cudaError_t pack_int32(const int32_t *in, uint32_t *planes, int rows, int K, int bits, cudaStream_t stream);
cudaError_t pack_int4(const void *in, uint32_t *planes, int rows, int K, int bits, cudaStream_t stream);
cudaError_t quantize_pack_half(const __half *in, const float *scale, uint32_t *planes, int rows, int K, int bits, int mode,
                               cudaStream_t stream);

// ---- wquant.cu
cudaError_t quantize_weights(const __half *w, uint32_t *planes, __half *scale, uint8_t *zero, int N, int K, int bits, int group_size, int symmetric,
                             cudaStream_t stream);

// Largest dynamic shared-memory size already opted in for one kernel, per device (the attribute is per device and
// function).  One instance per kernel instantiation and host thread: `static thread_local SmemOptIn done;`
struct SmemOptIn {
    static constexpr int kMaxDevices = 64;
    size_t bytes[kMaxDevices] = {};
    template <typename Kernel>
    cudaError_t ensure(Kernel kern, size_t need)
    {
        int dev = 0;
        cudaError_t e = cudaGetDevice(&dev);
        if (e != cudaSuccess)
            return e;
        const bool tracked = dev >= 0 && dev < kMaxDevices;
        if (tracked && need <= bytes[dev])
            return cudaSuccess;
        e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)need);
        if (e == cudaSuccess && tracked)
            bytes[dev] = need;
        return e;
    }
};

// ---- xprep.cu
// zero != NULL: the codes written are code - zero[row][k / zero_group] (the caller guarantees that this fits int8)
cudaError_t unpack_i8(const uint32_t *planes, void *out, int rows, int K, int bits, int is_signed, cudaStream_t stream,
                      const uint8_t *zero = nullptr, int zero_group = 0);
// fp16 activations -> int8 codes [rows][K] (static scale, truncation: the FasterTransformer wrapper's quantiser)
cudaError_t quantize_codes(const void *in_half, const float *scale, void *out, int rows, int K, int bits, cudaStream_t stream);
// both operands of a GEMM (same K) in one launch
cudaError_t unpack_pair_i8(const uint32_t *planes_a, void *out_a, int rows_a, int bits_a, int signed_a, const uint32_t *planes_b, void *out_b,
                           int rows_b, int bits_b, int signed_b, int K, cudaStream_t stream, const uint8_t *zero_b = nullptr,
                           int zero_group = 0);
// Bytes of one decode-route activation record (one per 128 input features): MT token tiles of 8.
__host__ __device__ constexpr int decode_record_bytes(int MT) { return 1024 * MT + 64; }

// ---- gemm_decode.cu (route ABQ_ROUTE_I8_MMA; taller problems run 16 rows per launch)
constexpr int kDecodeMaxSlices = 8;  // largest split-K factor (the workspace reserves that many partial slots)
// clear_counters: zero the split-K arrival counters now and wait for it (plans that are launched many times);
// otherwise the caller queues decode_clear_counters() on its stream before the launch (one-shot calls)
abq_status decode_plan(abq_gemm_state *st, bool clear_counters);
cudaError_t decode_clear_counters(const abq_gemm_state *st, cudaStream_t stream);
cudaError_t decode_launch(const abq_gemm_state *st, cudaStream_t stream);
size_t decode_workspace_bytes(int M, int N, int K);
// split-K scratch shared by both decode kernels: [tile counters][partial slots for kDecodeMaxSlices slices]
void decode_workspace_layout(int M, int N, size_t *off_partials, size_t *total);

// ---- gemm_stream.cu (route ABQ_ROUTE_I8_MMA over prepared weights, ABQ_FLAG_WEIGHTS_PREPARED + w_prepared)
bool stream_supported(const abq_gemm_params &p);
void decode_table_hints(const abq_gemm_params &p, int *warps, int *slices, int *ring, int *split); // tuned shape of the plane-reading kernel
size_t stream_prepared_bytes(const abq_gemm_params &p);
abq_status stream_plan(abq_gemm_state *st, bool clear_counters);
bool stream_planned(const abq_gemm_state *st);
cudaError_t stream_prepare_weights(const abq_gemm_state *st, cudaStream_t stream);
cudaError_t stream_launch(const abq_gemm_state *st, cudaStream_t stream);

// ---- gemm_b1.cu (route ABQ_ROUTE_B1_MMA)
abq_status b1_plan(abq_gemm_state *st);
cudaError_t b1_launch(const abq_gemm_state *st, cudaStream_t stream);

// ---- gemm_umma.cu (route ABQ_ROUTE_I8_UMMA)
abq_status umma_plan(abq_gemm_state *st);
cudaError_t umma_prepare_weights(const abq_gemm_state *st, cudaStream_t stream);
cudaError_t umma_launch(const abq_gemm_state *st, cudaStream_t stream);
size_t umma_workspace_bytes(int M, int N, int K);

// ---- api.cu helpers
// Encodes a tiled TMA descriptor through the driver entry point (no link-time libcuda dependency).
// dims/strides innermost first; strides in bytes for dimensions 1..rank-1.
enum TmapSwizzle { TMAP_SWIZZLE_NONE = 0, TMAP_SWIZZLE_64B = 2, TMAP_SWIZZLE_128B = 3 };
enum TmapDtype { TMAP_U8 = 0, TMAP_U32 = 1 };
bool encode_tmap(void *out128, TmapDtype dtype, int rank, const void *base, const uint64_t *dims, const uint64_t *strides_bytes,
                 const uint32_t *box, TmapSwizzle swizzle);
void set_last_cuda_error(cudaError_t e);
int env_int(const char *name, int fallback);

} // namespace abq
