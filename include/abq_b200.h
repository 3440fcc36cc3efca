/*
 * abq_b200.h -- C ABI of the B200 (sm_100a) arbitrary-bit quantized GEMM engine.
 *
 * The library computes D = X * W^T where X (M x K, p-bit codes) and W (N x K, q-bit codes) are
 * stored as bit-planes of 32-bit words:
 *
 *     plane word  P[b][row][kw]   (b < bits, row < rows, kw < K/32)
 *     bit (31 - j) of that word = bit b of the code of element (row, 32*kw + j)
 *
 * Unsigned code value = sum_b 2^b bit_b.  Signed: the top plane has weight -2^(bits-1).
 * K must be a multiple of 128.  This is the storage format of the reference engine
 * (engine/common/pack.cu:46-64, engine/mma_any/aq_bmma_kernel.h:121-127); weights arrive already
 * packed, activations are packed (or quantised and packed) per call.
 *
 * All pointers are device pointers unless stated otherwise.  No entry point allocates memory: scratch is a
 * caller-owned workspace (abq_gemm_static_scratch alone uses a fixed array that is part of the library's device
 * code instead).  All launches are asynchronous on the stream given.
 * Every entry point returns an abq_status; 0 is success.  There is no CPU fallback: if no usable
 * GPU kernel exists for a request the call fails with ABQ_ERR_UNSUPPORTED.
 *
 * Each declaration cites the reference interface it replaces (path inside the reference repo), or says that the
 * reference has no counterpart.
 */
#ifndef ABQ_B200_H
#define ABQ_B200_H

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define ABQ_API __attribute__((visibility("default")))
#else
#define ABQ_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

/* A CUDA stream handle (cudaStream_t) passed as an opaque pointer so that C callers need no CUDA headers. */
typedef void *abq_stream_t;

typedef enum abq_status {
    ABQ_OK = 0,
    ABQ_ERR_INVALID_ARG = 1,   /* null pointer, bad shape (K % 128 != 0, bits outside 1..8, ...) */
    ABQ_ERR_UNSUPPORTED = 2,   /* valid request with no kernel (e.g. bias != 0) */
    ABQ_ERR_WORKSPACE = 3,     /* workspace missing or smaller than abq_gemm_workspace_bytes() */
    ABQ_ERR_CUDA = 4,          /* a CUDA runtime/driver call failed; see abq_last_cuda_error() */
    ABQ_ERR_NOT_INITIALIZED = 5, /* abq_gemm_exec on a state that abq_gemm_init did not complete */
    ABQ_ERR_DEVICE_TIMEOUT = 6 /* reported through the device status word: a bounded wait expired */
} abq_status;

typedef enum abq_out_dtype {
    ABQ_OUT_INT32 = 0, /* raw plane-accumulated int32, as the reference engine writes */
    ABQ_OUT_FP16 = 1   /* fused dequantisation to IEEE half */
} abq_out_dtype;

typedef enum abq_scale_mode {
    ABQ_SCALE_NONE = 0,          /* int32 output only */
    ABQ_SCALE_TENSOR_COMPAT = 1, /* D = half(int acc) * C[0]: the FasterTransformer copy's epilogue */
    ABQ_SCALE_CHANNEL = 2,       /* D = x_scale[m] * w_scale[n] * (acc - w_zero[n] * sum_k x[m][k]) */
    ABQ_SCALE_GROUP = 3          /* same with one scale/zero per run of group_size input features */
} abq_scale_mode;

typedef enum abq_route {
    ABQ_ROUTE_AUTO = 0,     /* M <= 32 (16 with prepared weights): I8_MMA; otherwise I8_UMMA (per-group scales it cannot fold: I8_MMA) */
    ABQ_ROUTE_B1_MMA = 1,   /* legacy mma.sync b1 AND+POPC over stacked planes (route A) */
    ABQ_ROUTE_I8_MMA = 2,   /* planes recombined in registers, mma.sync s8/u8, TMA-fed, split-K (decode); M > 16 runs 16 rows per launch */
    ABQ_ROUTE_I8_UMMA = 3   /* planes recombined to int8 tiles, tcgen05.mma kind::i8 in TMEM (route B) */
} abq_route;

enum {
    /* Launch with programmatic dependent launch so that consecutive GEMMs overlap.  The decode kernels then request
     * their first weights BEFORE waiting for the kernel launched ahead of them on the stream: W (or w_prepared) must
     * be complete before that kernel starts -- do not launch a PDL GEMM directly behind the kernel that writes its
     * weights (abq_pack_int32, abq_gemm_prepare_weights, an upload); X, scales and D are read / written after the wait. */
    ABQ_FLAG_PDL = 1,
    /* The weights have been brought into the form the route computes on, once, by abq_gemm_prepare_weights; later calls
     * skip that work.  For weights that stay the same from call to call (a model's linear layers).
     *   Route I8_UMMA: the int8 expansion of W sits in this plan's workspace (a workspace of its own, which nothing
     *     else overwrites): abq_gemm_exec expands the activations only.
     *   Route I8_MMA (decode shapes): params.w_prepared points to abq_gemm_prepared_weight_bytes() bytes owned by the
     *     caller; abq_gemm_prepare_weights re-orders the planes W (and per-group scales / zero points) into it -- the
     *     same bits in the order the kernel consumes them -- and abq_gemm_exec reads w_prepared instead of W.  One
     *     prepared copy serves every token count up to 16 with the same scale mode and signedness.  Where
     *     abq_gemm_prepared_weight_bytes() is 0 (widths 1, 5, 6, 7; unsigned 8-bit activations) or w_prepared is
     *     NULL the flag is ignored on this route and W is read. */
    ABQ_FLAG_WEIGHTS_PREPARED = 2,
    /* X points to fp16 activations [M][K] instead of planes; the call quantises them itself exactly as the
     * FasterTransformer wrapper's pack does (abq_gemm_wrapper.cu:29-54): code = (int)(half(x) * half(x_quant_scale[0])),
     * truncated, unclamped, the low x_bits bits kept (x_signed must be 1).  Saves the pack launch and the round trip
     * through planes; the result is bit-identical to abq_quantize_pack_half (mode 0) followed by the GEMM. */
    ABQ_FLAG_X_HALF = 4
};

/*
 * All-reduce fused into a row-parallel GEMM (decode shapes, prepared weights, fp16 output): D receives the SUM over the
 * ranks of one node of what each rank's GEMM alone would have written (its fp16 partial), added in rank order in fp32 --
 * the same bits on every rank.  Replaces, together with the GEMM, the ncclAllReduce that the reference's FasterTransformer
 * fork issues after the attention output and FFN down projections (TensorParallelGptContextAttentionLayer.cc:50-53,
 * TensorParallelSiluFfnLayer.cc:53-57).  How: as a CTA finishes its 16-row tiles it stores its partial straight into every
 * rank's receive buffer (peer stores over NVLink), raises a flag per tile in every rank's flag array, waits (bounded,
 * status_word) for the other ranks' flags of the same tiles and adds what they stored.  No separate kernel, no
 * round trip for the data.  Buffers alternate with the parity of a device-side call counter, so a rank that runs ahead
 * writes the other half; a launch replays inside a CUDA graph.
 *   recv[r], flags[r]  rank r's receive buffer / flag array as mapped into THIS process (peer mappings, e.g. torch symmetric
 *                      memory); entries [rank] are the local ones.  recv: 2 * world * rows_cap * N fp16
 *                      ([parity][source rank][token][feature]); flags: 2 * world * ceil(N / 16) uint32, zero before first use
 *   counter            local, two uint32, zero before first use (calls completed, CTA ticket); one per call site
 *   rows_cap           token rows the receive buffers were sized for (>= M)
 * Every rank must run the same sequence of fused GEMMs per call site.  Only plain peer stores and loads are used.
 */
typedef struct abq_fused_allreduce {
    int world, rank; /* 2..8 ranks */
    void *recv[8];
    uint32_t *flags[8];
    uint32_t *counter;
    int rows_cap;
} abq_fused_allreduce;

/*
 * Problem description.  The first eight fields are the reference's launch arguments in the
 * reference's order (engine/mma_any/aq_bmma_op.h:24-31 `AqBMMAOpState::Argument_t`:
 * M, N, K, X, W, C, D, bias); the rest extends them.
 */
typedef struct abq_gemm_params {
    int M, N, K;
    const void *X;  /* uint32 planes [x_bits][M][K/32] (fp16 [M][K] with ABQ_FLAG_X_HALF) */
    const void *W;  /* uint32 planes [w_bits][N][K/32] */
    const void *C;  /* ABQ_SCALE_TENSOR_COMPAT: one fp16 scale; otherwise unused (reference: `half *C`) */
    void *D;        /* int32 [M][N] or fp16 [M][N], row-major */
    int bias;       /* must be 0: the reference asserts !bias (aq_bmma_op.h:79) */

    int x_bits, w_bits;     /* 1..8 each */
    int x_signed, w_signed; /* the reference has one SIGNED flag for both (common/base.h QuantType) */
    int out_dtype;          /* abq_out_dtype */
    int scale_mode;         /* abq_scale_mode */
    int group_size;         /* ABQ_SCALE_GROUP: multiple of 128 dividing K */
    const void *w_scale;    /* fp16 [N] (CHANNEL) or [N][K/group_size] (GROUP) */
    const uint8_t *w_zero;  /* optional zero points, same shape as w_scale, NULL = 0; each must lie in the code range,
                               0 .. 2^w_bits - 1: the kernels' exactness bounds (int8 operands, the 2^22 bound of the
                               integer-to-float step) assume it and nothing checks device data */
    const float *x_scale;   /* optional per-token fp32 scale [M], NULL = 1 */
    int route;              /* abq_route */
    int flags;              /* ABQ_FLAG_* */
    void *workspace;        /* >= abq_gemm_workspace_bytes(), 256-byte aligned */
    size_t workspace_bytes;
    int *status_word;       /* optional device int, set non-zero by a kernel whose bounded wait expired */
    const float *x_quant_scale; /* ABQ_FLAG_X_HALF: device float, the static activation scale */
    void *w_prepared;           /* ABQ_FLAG_WEIGHTS_PREPARED on route I8_MMA: the re-ordered weights, 16-byte aligned */
    const abq_fused_allreduce *allreduce; /* optional (host pointer, copied by abq_gemm_init): sum D over the ranks inside the
                                             GEMM; plans that cannot do it answer ABQ_ERR_UNSUPPORTED */
    const void *residual;   /* optional fp16 [M][N] (fp16 output, route I8_MMA; other plans answer ABQ_ERR_UNSUPPORTED):
                               D = half(result) + residual, the fp16 add a separate residual kernel would do after the GEMM
                               (after the sum over the ranks when `allreduce` is set); may alias neither X nor D */
} abq_gemm_params;

/*
 * Launch plan produced by abq_gemm_init and consumed by abq_gemm_exec.  Plain data, copyable, no
 * ownership.  Replaces `AqBMMAOpState` (engine/mma_any/aq_bmma_op.h:19-32).
 */
typedef struct abq_gemm_state {
    abq_gemm_params p;
    int init_success;  /* reference: `bool initSuccess` */
    int route;         /* route chosen (abq_route, never AUTO) */
    int grid[3];
    int block[3];
    int cluster;       /* split-K factor == cluster size along K (decode route) */
    size_t shared_mem_size;
    int tile[4];       /* route specific tile description */
    unsigned long long tmap[3][16]; /* TMA tensor maps (128 B each), route specific */
    abq_fused_allreduce ar;         /* copy of *p.allreduce (world == 0: none) */
} abq_gemm_state;

/* Bytes of caller-owned scratch a GEMM of this shape may need (route AUTO: the maximum over routes). */
ABQ_API size_t abq_gemm_workspace_bytes(int M, int N, int K, int x_bits, int w_bits, int route);

/*
 * Plan a GEMM: validates, picks the route and tile, encodes TMA descriptors.  Host work, except that a
 * decode-shape plan which splits K over CTAs clears its arrival counters (the first 4 * ceil(N / 16) bytes of the
 * workspace) and waits for that: call it outside stream capture and not while a GEMM on the same workspace is
 * running; launches leave the counters cleared, so plans may share a workspace.  Replaces `AqBMMAInitFn_t` / `AqBWMMAInitFn_t`
 * (engine/mma_any/aq_bmma_op.h:141-151,163; aq_wmma_op.h) and the per-config
 * `AqBMMA_..._InitFn` globals (engine/common/base.h:144-166): tile shape is chosen here, not by name.
 */
ABQ_API abq_status abq_gemm_init(const abq_gemm_params *params, abq_gemm_state *state);

/*
 * Launch a planned GEMM on `stream`.  Replaces `AqBMMAExecFn_t` (aq_bmma_op.h:153-164) and
 * `launchWmmaAnyKernel` (engine/wmma_any/wmma_any.h:30-38).
 */
ABQ_API abq_status abq_gemm_exec(const abq_gemm_state *state, abq_stream_t stream);

/* init + exec in one call (what the FasterTransformer wrapper does per linear layer,
 * fastertransformer/src/fastertransformer/kernels/abqgemm/abq_gemm_wrapper.cu:125-137). */
ABQ_API abq_status abq_gemm(const abq_gemm_params *params, abq_stream_t stream);

/*
 * Value tensor -> bit-planes.  `in` holds one int32 per code, row-major [rows][K]; only the low
 * `bits` bits are used.  Replaces `launch_pack` (engine/common/pack.h:23-24, pack.cu:93-103) and
 * `ABQGEMMWrapper::pack(const int*, ...)` (abq_gemm_wrapper.cu:71-77).
 */
ABQ_API abq_status abq_pack_int32(const int32_t *in, void *planes, int rows, int K, int bits, abq_stream_t stream);

/*
 * Nibble-packed 4-bit codes (8 per 32-bit word, first element in the most significant nibble)
 * -> bit-planes.  Replaces `launch_pack4` (engine/common/pack.h:20-21, pack.cu:73-84).
 */
ABQ_API abq_status abq_pack_int4(const void *in, void *planes, int rows, int K, int bits, abq_stream_t stream);

/*
 * fp16 activations -> integer codes -> bit-planes in one pass.
 *   mode 0 (compat): code = (int)(half(x) * half(scale[0])), truncating, unclamped: bit-exact twin
 *                    of `pack_half` (abq_gemm_wrapper.cu:29-54, called from :62-69).
 *   mode 1 (rtn):    code = clamp(rint(x / scale[row]), -2^(bits-1), 2^(bits-1)-1), per-token
 *                    scale (the dynamic per-token quantiser of algorithm/quantize/quantizer.py:111-159).
 * `scale` is a device pointer to 1 (mode 0) or `rows` (mode 1) floats.
 */
ABQ_API abq_status abq_quantize_pack_half(const void *in_half, const float *scale, void *planes, int rows, int K,
                                  int bits, int mode, abq_stream_t stream);

/*
 * Quantise-on-load: fp16 weights [N][K] -> unsigned w-bit codes written as bit-planes [bits][N][K/32] (the layout
 * abq_pack_int32 writes), fp16 scale and u8 zero point per output channel (group_size 0: [N]) or per run of group_size
 * input features (a multiple of 32 dividing K: [N][K/group_size]); dequantised weight = (code - zero) * scale.  Min/max
 * calibration and code rule of the reference's quantiser (algorithm/quantize/quantizer.py:111-132, 149-179, without
 * learnable clipping), in fp32; `symmetric` picks its symmetric variant (quantizer.py:163-167).  Codes and zero points are
 * clamped into 0 .. 2^bits - 1, the range the planes can hold (the reference's 1/2-bit "bit balance" allows 2^bits).
 * The reference has no GPU counterpart: its FasterTransformer loader expects planes packed offline
 * (LlamaDecoderLayerWeight.cc:377-403) and random-initialises what it does not find.
 */
ABQ_API abq_status abq_quantize_weights_half(const void *w_half, int N, int K, int bits, int group_size, int symmetric, void *planes,
                                             void *scale_half, uint8_t *zero, abq_stream_t stream);

/*
 * Bytes of the prepared copy of W that a decode-shape plan (route I8_MMA) with ABQ_FLAG_WEIGHTS_PREPARED reads through
 * params->w_prepared: the planes' own w_bits * N * K / 8 bytes (N rounded up to 16) plus, with per-group scales, 4
 * bytes per row and 128 input features.  Depends on N, K, w_bits, scale_mode, x_bits / x_signed only.  0 = this problem
 * has no prepared form on that route.  No reference counterpart.
 */
ABQ_API size_t abq_gemm_prepared_weight_bytes(const abq_gemm_params *params);

/*
 * Bring the weights of a planned GEMM with ABQ_FLAG_WEIGHTS_PREPARED into the form its route computes on, once: the
 * int8 expansion in the plan's workspace (route I8_UMMA) or the re-ordered copy in params.w_prepared (route I8_MMA).
 * A no-op returning ABQ_OK for plans that read the planes directly.  No reference counterpart: the reference
 * multiplies the planes themselves (its weights are packed offline into planes, engine/common/pack.cu, and that
 * format stays the input here).
 */
ABQ_API abq_status abq_gemm_prepare_weights(const abq_gemm_state *state, abq_stream_t stream);

/*
 * Sum of fp16 partial results over the ranks of one node, read out of the peers' memory (NVLink peer loads): what a
 * row-parallel linear layer needs after its GEMM.  Replaces the ncclAllReduce of the reference's FasterTransformer fork
 * (TensorParallelGptContextAttentionLayer.cc:50-53, TensorParallelSiluFfnLayer.cc:53-57) for decode-sized messages.
 *   bufs_dev     device array of `world` pointers: every rank's partial buffer as mapped into THIS process (peer
 *                mappings, e.g. torch symmetric memory `buffer_ptrs_dev`); bufs_dev[rank] is the local one, already
 *                written by earlier work on `stream`
 *   signals_dev  device array of `world` pointers to the ranks' signal pads; uint32 words signal_offset .. signal_offset +
 *                2 * world - 1 of every pad belong to this call site and are zero before first use
 *   out          local result, n_halves fp16 values (n_halves % 8 == 0); must not alias a partial buffer
 *   counter      two device uint32, zero before first use: the call count (lets a CUDA graph replay the launch) and a
 *                block ticket
 * Every rank adds in rank order in fp32: all ranks get the same bits.  The call returns (on the stream) only after every
 * peer has read this rank's buffer, so the buffer may be rewritten by whatever comes next, and one call site can be used
 * back to back.  The waits for the peers are bounded (status_word).  abq_fused_allreduce does the same sum inside the GEMM.
 *   residual     optional local fp16 array of n_halves values added to the sum (fp16 add of the rounded sum, as a separate
 *                residual kernel after the all-reduce would do); NULL for the plain sum
 */
ABQ_API abq_status abq_peer_allreduce_half(const void *const *bufs_dev, uint32_t *const *signals_dev, int rank, int world,
                                           int signal_offset, void *out, long n_halves, uint32_t *counter, int *status_word,
                                           const void *residual, abq_stream_t stream);

/*
 * The fp16 elementwise steps between the GEMMs of a decoder block, as single launches that join the programmatic-dependent-
 * launch chain: out[m][f] = SiLU(gate_up[m][f]) * gate_up[m][F + f] over a fused gate+up output [M][2F] (the reference's
 * FasterTransformer fork: genericActivation after the gate and up GEMMs, layers/FfnLayer.cc:407-421; SiLU in fp32, rounded to
 * fp16 before the product) and out = a + b (its residual adds).  F and n multiples of 8, pointers 16-byte aligned.
 */
ABQ_API abq_status abq_swiglu_half(const void *gate_up, void *out, int M, int F, abq_stream_t stream);
ABQ_API abq_status abq_add_half(const void *a, const void *b, void *out, long n, abq_stream_t stream);

/*
 * (Residual add ->) RMSNorm -> activation quantiser -> bit-planes in one launch, one read of the row.  Replaces the chain
 * the reference's FasterTransformer fork runs in front of every quantized GEMM: invokeGeneralAddBiasResidualPreLayerNorm /
 * invokeGeneralT5LayerNorm (fp16 output) followed by ABQGEMMWrapper::pack (kernels/abqgemm/abq_gemm_wrapper.cu:79-98).
 *   s = x (+ residual, fp16 add; written to sum_out_half when that is given)
 *   y = half((float(s) * rsqrt(mean(s^2) + eps)) * float(gamma))        gamma: fp16 [K]; written to y_out_half when given
 *   planes[bits][rows][K/32] = codes of y:  mode 0  (int)(y * half(scale[0]))              the wrapper's quantiser
 *                                           mode 1  clamp(rint(float(y) / scale[row]))     given per-token scales
 *                                           mode 2  as mode 1 with scale[row] = max|y| / (2^(bits-1) - 1), chosen here and
 *                                                   written to row_scale_out[rows] (the GEMM epilogue's x_scale)
 * The planes equal abq_quantize_pack_half applied to y bit for bit.  planes may be NULL (normalisation only).
 * K a multiple of 128, at most 16384; fp16 pointers 16-byte aligned.  Joins a programmatic-dependent-launch chain (gamma
 * must be complete before the preceding kernel starts).
 */
ABQ_API abq_status abq_rmsnorm_quantize_pack_half(const void *x_half, const void *residual_half, void *sum_out_half, const void *gamma_half,
                                                  float eps, const float *scale, float *row_scale_out, void *planes, void *y_out_half,
                                                  int rows, int K, int bits, int mode, abq_stream_t stream);

/* Bit-planes -> int8 codes, row-major [rows][K] (two's complement for signed; unsigned 8-bit codes are
 * stored as uint8).  Used by route B; exported because weight planes can be expanded once and cached. */
ABQ_API abq_status abq_unpack_int8(const void *planes, void *out_i8, int rows, int K, int bits, int is_signed,
                           abq_stream_t stream);

/*
 * abq_gemm for callers that cannot supply scratch memory.  No counterpart in the reference.
 *
 * Same contract as abq_gemm, except that params->workspace / workspace_bytes are ignored and that
 * ABQ_FLAG_WEIGHTS_PREPARED is refused (ABQ_ERR_INVALID_ARG) wherever the prepared weights would live in the workspace
 * (the shared array holds whatever the last call left): it is accepted only with route == ABQ_ROUTE_I8_MMA and a
 * w_prepared buffer, where the prepared copy is the caller's own and the scratch holds split-K partial sums only.
 * The scratch the chosen route needs is taken from one array
 * of ABQ_STATIC_SCRATCH_BYTES bytes in the library's device code: a GPU holds it from the moment the CUDA runtime
 * loads that code on it (with lazy loading: the first call on that GPU) until the process exits.  The call allocates nothing (no cudaMalloc, no
 * cudaFree, no allocating library routine), which is what a caller needs that runs inside a stream-ordered forward
 * pass with a workspace it does not size itself (the FasterTransformer linear layers give the GEMM wrapper only
 * x_bits * tokens * K / 8 bytes) and must not synchronise the device.
 *   - Problems whose abq_gemm_workspace_bytes() exceeds ABQ_STATIC_SCRATCH_BYTES are rejected with
 *     ABQ_ERR_WORKSPACE; use abq_gemm with a caller-owned workspace for those.
 *   - The first call on a device looks the array's address up (cudaGetSymbolAddress, with that device current).
 *     Make that first call outside any stream capture.
 *   - All calls on a device share the one array and it keeps what the last call left in it.  The kernels
 *     overwrite what they read before they read it, so nothing needs clearing, but two calls that overlap on the
 *     GPU (different streams, or graphs replayed concurrently) race on it: serialise them on one stream.
 */
#define ABQ_STATIC_SCRATCH_BYTES (16u << 20)
ABQ_API abq_status abq_gemm_static_scratch(const abq_gemm_params *params, abq_stream_t stream);

/* Text for a status code; cudaError_t of the last failing CUDA call in this thread (0 if none). */
ABQ_API const char *abq_status_string(abq_status s);
ABQ_API int abq_last_cuda_error(void);

/* Library / build identification, e.g. "abq_b200 0.1 sm_100a". */
ABQ_API const char *abq_version(void);

#ifdef __cplusplus
}
#endif
#endif /* ABQ_B200_H */
