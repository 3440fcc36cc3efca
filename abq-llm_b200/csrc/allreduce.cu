// Sum of the fp16 partial results of the row-parallel GEMMs over the ranks of one node, read straight out of the peers'
// memory (NVLink peer loads; no multimem, no library collective).  Replaces the ncclAllReduce that the reference's
// FasterTransformer fork issues after the attention output and the FFN down projections
// (TensorParallelGptContextAttentionLayer.cc:50-53, TensorParallelSiluFfnLayer.cc:53-57) for the small messages of a
// decode step, where the latency of a collective call, not its bandwidth, is what costs.
//
// One-shot: every rank's partial lies in a buffer that all ranks have mapped (bufs[r] on every rank); a rank tells each
// peer that its buffer is written (a flag in the peer's signal pad, release at system scope), waits for the peers'
// flags in its own pad (acquire, bounded), then reads all buffers and adds them in rank order in fp32, so every rank
// gets the same bits.  The flag value is a call counter kept on the device, so a CUDA graph can replay the launch.
// Several blocks share the message (remote loads are latency-bound: more of them in flight); block 0 flags the peers,
// every block waits for the peers' flags, and the last block to finish advances the counter.
// The call ends with a second flag round ("I have read your buffer"): a rank leaves the kernel only when every peer has
// finished reading its partial, so whatever follows on its stream may overwrite the buffer at once -- a call site can be
// used back to back -- and a flag can never be a call ahead of the one a rank is waiting for (it waits for equality).
#include <cuda_fp16.h>

#include "abq_common.cuh"
#include "abq_kernels.h"

namespace abq {

constexpr int kAllreduceThreads = 1024;

__global__ void __launch_bounds__(kAllreduceThreads) peer_allreduce_kernel(const __half *const *bufs, uint32_t *const *signals, int rank,
                                                                           int world, int signal_offset, __half *out, long n, uint32_t *counter, int *status,
                                                                           const __half *residual)
{
    // counter[0]: calls completed; counter[1]: blocks of this call that have finished
    __shared__ uint32_t s_epoch;
    if (threadIdx.x == 0)
        s_epoch = *reinterpret_cast<volatile uint32_t *>(counter) + 1; // (only the last block of a call writes it, after all have read it)
    __syncthreads();
    const uint32_t epoch = s_epoch;
    if ((int)threadIdx.x < world && (int)threadIdx.x != rank) {
        const int peer = threadIdx.x;
        if (blockIdx.x == 0) {
            // everything earlier in the stream (the GEMM that wrote bufs[rank]) is complete: publish
            __threadfence_system();
            uint32_t *theirs = signals[peer] + signal_offset + rank; // my column of the peer's pad
            asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(theirs), "r"(epoch) : "memory");
        }
        const uint32_t *mine = signals[rank] + signal_offset + peer;
        const unsigned long long t0 = globaltimer_ns();
        for (;;) {
            uint32_t v;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
            if (v == epoch)
                break;
            if (globaltimer_ns() - t0 > kWaitLimitNs) { // the peer never arrived: record it and carry on (the sum is then void)
                if (status)
                    atomicOr(status, STATUS_TIMEOUT_PIPE);
                break;
            }
        }
    }
    __syncthreads();
    for (long i = ((long)blockIdx.x * kAllreduceThreads + threadIdx.x) * 8; i < n; i += (long)gridDim.x * kAllreduceThreads * 8) { // 16 bytes
        float acc[8] = { 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f };
        for (int r = 0; r < world; ++r) {
            const uint4 v = __ldcv(reinterpret_cast<const uint4 *>(bufs[r] + i)); // no stale cached copy of a peer's line
            const __half2 *h = reinterpret_cast<const __half2 *>(&v);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 f = __half22float2(h[e]);
                acc[2 * e] += f.x;
                acc[2 * e + 1] += f.y;
            }
        }
        uint4 o;
        __half2 *oh = reinterpret_cast<__half2 *>(&o);
#pragma unroll
        for (int e = 0; e < 4; ++e)
            oh[e] = __floats2half2_rn(acc[2 * e], acc[2 * e + 1]);
        if (residual) { // the fp16 add of a residual kernel that would otherwise follow
            const uint4 rv = *reinterpret_cast<const uint4 *>(residual + i);
            const __half2 *rh = reinterpret_cast<const __half2 *>(&rv);
#pragma unroll
            for (int e = 0; e < 4; ++e)
                oh[e] = __hadd2(oh[e], rh[e]);
        }
        *reinterpret_cast<uint4 *>(out + i) = o;
    }
    __syncthreads();
    bool last = gridDim.x == 1; // a lone block needs no ticket
    if (threadIdx.x == 0 && gridDim.x > 1) {
        const uint32_t done = atomicAdd(counter + 1, 1u);
        last = done == gridDim.x - 1; // every block of this call has read the counter and the peers' buffers
    }
    if (threadIdx.x == 0)
        s_epoch = last ? 1u : 0u;
    __syncthreads();
    if (s_epoch == 0u)
        return;
    // ---- closing round, by the block that finished last: tell the peers that their buffers have been read, wait until
    // they have read ours
    if ((int)threadIdx.x < world && (int)threadIdx.x != rank) {
        const int peer = threadIdx.x;
        uint32_t *theirs = signals[peer] + signal_offset + world + rank;
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(theirs), "r"(epoch) : "memory");
        const uint32_t *mine = signals[rank] + signal_offset + world + peer;
        const unsigned long long t0 = globaltimer_ns();
        for (;;) {
            uint32_t v;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
            if (v == epoch)
                break;
            if (globaltimer_ns() - t0 > kWaitLimitNs) {
                if (status)
                    atomicOr(status, STATUS_TIMEOUT_PIPE);
                break;
            }
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        counter[1] = 0;
        __threadfence();
        counter[0] = epoch;
    }
}

cudaError_t peer_allreduce(const void *const *bufs_dev, uint32_t *const *signals_dev, int rank, int world, int signal_offset, void *out,
                           long n_halves, uint32_t *counter, int *status, const void *residual, cudaStream_t stream)
{
    long blocks = (n_halves / 8 + kAllreduceThreads - 1) / kAllreduceThreads; // one 16-byte piece per thread where that needs <= 32 blocks
    blocks = blocks < 1 ? 1 : (blocks > 32 ? 32 : blocks);
    peer_allreduce_kernel<<<(unsigned)blocks, kAllreduceThreads, 0, stream>>>(reinterpret_cast<const __half *const *>(bufs_dev), signals_dev, rank, world,
                                                               signal_offset, reinterpret_cast<__half *>(out), n_halves, counter, status,
                                                               reinterpret_cast<const __half *>(residual));
    return cudaGetLastError();
}

} // namespace abq

extern "C" abq_status abq_peer_allreduce_half(const void *const *bufs_dev, uint32_t *const *signals_dev, int rank, int world,
                                              int signal_offset, void *out, long n_halves, uint32_t *counter, int *status_word,
                                              const void *residual, abq_stream_t stream)
{
    if (!bufs_dev || !signals_dev || !out || !counter || world < 1 || world > 32 || rank < 0 || rank >= world || n_halves <= 0 ||
        n_halves % 8 != 0 || signal_offset < 0 || ((reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(residual)) & 15))
        return ABQ_ERR_INVALID_ARG;
    cudaError_t e = abq::peer_allreduce(bufs_dev, signals_dev, rank, world, signal_offset, out, n_halves, counter, status_word, residual,
                                        reinterpret_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) {
        abq::set_last_cuda_error(e);
        return ABQ_ERR_CUDA;
    }
    return ABQ_OK;
}
