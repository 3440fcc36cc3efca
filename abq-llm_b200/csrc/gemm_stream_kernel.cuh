// Decode-shape GEMM (up to 16 rows per launch) over weights in the library's own "stream" layout: the same bits as the
// reference's bit-planes (engine/common/pack.cu:46-64), re-ordered once at load time (prepare_stream_kernel below) so
// that the kernel that runs every step spends its instructions on arithmetic instead of on un-shuffling planes.
//
// Layout.  The weight matrix is cut into units of 16 output rows x 128 input features; a unit is Q * 256 bytes of codes
// followed (when scales come per group) by 64 bytes of parameters, and the units of a 16-row tile follow one another
// along K, tile after tile.  Inside a unit, lane l = 4 g + t of a warp owns rows g and g + 8 and the features
// 32 t .. 32 t + 31; its codes sit where the lane reads them with 16-byte loads and are packed so that one AND (for
// some fields of the 3-bit format a shift, AND, OR) per register yields the A fragments of mma.sync.m16n8k32 as byte
// values times a power of two; fragments with different powers go to different accumulator sets, merged exactly when
// the sets are folded.  The 64 parameter bytes are, per row, the fp32 bits of the group's fp16 scale with the zero
// point (plus the offset of two's-complement codes) in the low mantissa bits, which an fp16 value leaves zero.
//
// Kernel.  A CTA owns a contiguous range of tiles, i.e. one contiguous byte range of the stream; its warps deal the
// range among themselves in chunks of a few units and every warp pulls its chunks through a private ring with plain bulk
// copies (cp.async.bulk, no tensor map), refilling a slot as soon as it is consumed.  Weight requests go out before the
// wait on the previous kernel (programmatic dependent launch), and the kernel is shaped so that two CTAs fit on an SM:
// while one GEMM computes, the next one's CTAs are already resident with their first chunks in shared memory.
// The activations are expanded once per CTA into byte "records" (the B fragments) plus per-unit code sums.
// With few tokens the eight columns of the MMA would mostly multiply padding; instead column c holds token c % MP of
// unit (c / MP) of a block of GS = 8 / MP consecutive units (their B fragments are zero elsewhere), so the fold of the
// integer accumulators into fp32 -- the expensive part of group-wise scales -- happens once per GS units.
// Partial sums of the warps that share a tile meet in shared memory after one barrier and are added in warp order.
//
// Covers, for prepared weights, what the reference does with plane-stacked 1-bit MMAs and a shared-memory
// shift-accumulate epilogue (engine/mma_any/aq_bmma_kernel.h:109-271, 485-580; fp16 scalar epilogue of the
// FasterTransformer copy, fastertransformer/.../abqgemm/mma_any/aq_bmma_kernel.h:474-524).
#pragma once
#include <cuda.h>
#include <cstring>
#include <type_traits>

#include "abq_common.cuh"
#include "abq_kernels.h"
#include "xbytes.cuh"

namespace abq {

constexpr int kStreamMaxWarps = 16;
constexpr int kStreamMaxRing = 8;
constexpr uint32_t kZeroMask = 0x1fffu; // low mantissa bits of the packed (scale, zero) word that hold the zero point

// Fused all-reduce (abq_fused_allreduce): every rank's receive buffer and flag array as mapped here.
struct StreamAllreduce {
    int world, rank, rows_cap, row0; // row0: first token row of this launch within the receive buffers
    __half *recv[8];
    uint32_t *flags[8];
    uint32_t *counter;
};

struct StreamArgs {
    int M, N, K;
    int tiles;           // ceil(N / 16)
    int uw;              // input features per unit: 128, or 64 when the scale groups are 64 wide
    int units;           // K / uw: units per tile in the stream
    int unit_bytes;      // Q * 2 * uw (+ 64 with group parameters)
    int slices;          // K split over CTAs (1 unless the records of all K do not fit in shared memory)
    int units_per_slice; // multiple of cu
    int ctas_per_slice;
    int cu;              // units per chunk (multiple of GS)
    int ring;            // chunks per warp ring
    int prefill;         // chunks per warp requested before the wait on the previous kernel (the rest right after it)
    int nw;              // warps per CTA (a power of two)
    // what the host can work out once instead of every thread at every launch (each of these is an integer division there):
    int nw_shift;            // log2(nw)
    int tiles_q, tiles_r;    // tiles / ctas_per_slice and the remainder: the first tiles_r CTAs of a slice take one tile more
    int max_tiles;           // ceil(tiles / ctas_per_slice)
    int cpt_full;            // chunks per tile of a slice with all its units_per_slice units
    uint32_t rec_magic;      // idx / (units_per_slice * uw / 32) == umulhi(idx, rec_magic) for the record items
    uint32_t per_tile_magic; // tid / (16 * M) == umulhi(tid, per_tile_magic)
    uint32_t cpt_magic;      // c / cpt_full == umulhi(c, cpt_magic) for the chunk indices of a CTA
    const uint8_t *Wp;   // weights in stream layout
    const uint32_t *X;   // activation planes [x_bits][rows][K/32], first row of this launch (fp16 [rows][K] with x_qscale)
    size_t x_plane_words;
    const float *x_qscale;
    int x_bits, x_signed;
    int *counters;  // slices > 1: one arrival counter per tile, zero before the launch, left zero after it
    int *partials;  // slices > 1: [slice][tile][token][16 rows]
    void *D;
    const __half *w_scale; // per-channel mode only (group parameters travel in the stream)
    const uint8_t *w_zero;
    const float *x_scale;
    const __half *C;
    int out_dtype, scale_mode, w_signed;
    int *status;
    const __half *residual; // not null: added (fp16) to the fp16 result before it is stored
    StreamAllreduce ar; // world <= 1: none
};


// ------------------------------------------------------------------------------------------ formats
// StreamFormat<Q>: how the codes of one lane (rows g and g + 8, 32 features each) are packed, and how they come back.
//   code(j, a, y): byte y of A register a (a0: row g low half, a1: row g + 8 low half, a2: row g high half, a3: row g + 8
//   high half) of MMA step j of the unit = the row's code at feature 32 t + 31 - 8 y - (2 j + (a >> 1)).
//   pack():   the codes of a lane as bytes c[row 0/1][s = 2 j + h] (byte y in bits 8y..8y+7) -> its kWords words
//   expand(): shared memory -> R[j][a] = code bytes * 2^(kShift * set_of(j))
template <int Q, int UW = 128>
struct StreamFormat;

template <>
struct StreamFormat<2, 128> {
    static constexpr int kSteps = 4;
    static constexpr int kWords = 4, kSets = 2, kShift = 2;
    __host__ __device__ static constexpr int set_of(int j) { return j & 1; }
    __device__ static void pack(const uint32_t (&c)[2][8], uint32_t (&w)[kWords])
    {
#pragma unroll
        for (int a = 0; a < 4; ++a) {
            w[a] = 0;
#pragma unroll
            for (int j = 0; j < 4; ++j)
                w[a] |= c[a & 1][2 * j + (a >> 1)] << (2 * j);
        }
    }
    __device__ static __forceinline__ void expand(const uint8_t *unit, int lane, uint32_t (&R)[4][4])
    {
        const uint4 v = *reinterpret_cast<const uint4 *>(unit + lane * 16);
        const uint32_t w[4] = { v.x, v.y, v.z, v.w };
#pragma unroll
        for (int a = 0; a < 4; ++a) {
            const uint32_t hi = w[a] >> 4;
            R[0][a] = w[a] & 0x03030303u;
            R[1][a] = w[a] & 0x0c0c0c0cu;
            R[2][a] = hi & 0x03030303u;
            R[3][a] = hi & 0x0c0c0c0cu;
        }
    }
};

template <>
struct StreamFormat<4, 128> {
    static constexpr int kSteps = 4;
    static constexpr int kWords = 8, kSets = 2, kShift = 4;
    __host__ __device__ static constexpr int set_of(int j) { return j & 1; }
    __device__ static void pack(const uint32_t (&c)[2][8], uint32_t (&w)[kWords])
    {
#pragma unroll
        for (int jj = 0; jj < 2; ++jj)
#pragma unroll
            for (int a = 0; a < 4; ++a)
                w[jj * 4 + a] = c[a & 1][4 * jj + (a >> 1)] | (c[a & 1][4 * jj + 2 + (a >> 1)] << 4);
    }
    __device__ static __forceinline__ void expand(const uint8_t *unit, int lane, uint32_t (&R)[4][4])
    {
#pragma unroll
        for (int jj = 0; jj < 2; ++jj) {
            const uint4 v = *reinterpret_cast<const uint4 *>(unit + jj * 512 + lane * 16);
            const uint32_t w[4] = { v.x, v.y, v.z, v.w };
#pragma unroll
            for (int a = 0; a < 4; ++a) {
                R[2 * jj][a] = w[a] & 0x0f0f0f0fu;
                R[2 * jj + 1][a] = w[a] & 0xf0f0f0f0u;
            }
        }
    }
};

// Three bits: eight codes of a byte lane in three bytes.  Slot s' of a row holds the code of step/half (j, h) with
// slot_of(j, h) below; slots 0, 3, 6, 2 come out times 1, slots 1, 4, 7, 5 times 8.
//   A = c0 | c1 << 3 | (c2 & 3) << 6;  B = c3 | c4 << 3 | (c5 & 3) << 6;  C = c6 | c7 << 3 | (c2 >> 2) << 6 | (c5 >> 2) << 7
template <>
struct StreamFormat<3, 128> {
    static constexpr int kSteps = 4;
    static constexpr int kWords = 6, kSets = 2, kShift = 3;
    __host__ __device__ static constexpr int set_of(int j) { return j >> 1; }
    __host__ __device__ static constexpr int slot_of(int j, int h)
    {
        return j == 0 ? (h ? 3 : 0) : j == 1 ? (h ? 2 : 6) : j == 2 ? (h ? 4 : 1) : (h ? 5 : 7);
    }
    __device__ static void pack(const uint32_t (&c)[2][8], uint32_t (&w)[kWords])
    {
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            uint32_t s[8];
#pragma unroll
            for (int j = 0; j < 4; ++j)
#pragma unroll
                for (int h = 0; h < 2; ++h)
                    s[slot_of(j, h)] = c[r][2 * j + h];
            const uint32_t A = s[0] | (s[1] << 3) | ((s[2] & 0x03030303u) << 6);
            const uint32_t B = s[3] | (s[4] << 3) | ((s[5] & 0x03030303u) << 6);
            const uint32_t C = s[6] | (s[7] << 3) | (((s[2] >> 2) & 0x01010101u) << 6) | (((s[5] >> 2) & 0x01010101u) << 7);
            // words 0..3 are the lane's 16-byte piece, words 4, 5 its 8-byte piece
            if (r == 0) {
                w[0] = A;
                w[1] = B;
                w[2] = C;
            } else {
                w[3] = A;
                w[4] = B;
                w[5] = C;
            }
        }
    }
    __device__ static __forceinline__ void expand(const uint8_t *unit, int lane, uint32_t (&R)[4][4])
    {
        const uint4 v = *reinterpret_cast<const uint4 *>(unit + lane * 16);
        const uint2 u = *reinterpret_cast<const uint2 *>(unit + 512 + lane * 8);
        const uint32_t abc[2][3] = { { v.x, v.y, v.z }, { v.w, u.x, u.y } };
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const uint32_t A = abc[r][0], B = abc[r][1], C = abc[r][2];
            uint32_t s[8];
            s[0] = A & 0x07070707u;
            s[1] = A & 0x38383838u;
            s[3] = B & 0x07070707u;
            s[4] = B & 0x38383838u;
            s[6] = C & 0x07070707u;
            s[7] = C & 0x38383838u;
            s[2] = ((A >> 6) & 0x03030303u) | ((C >> 4) & 0x04040404u);
            s[5] = ((B >> 3) & 0x18181818u) | ((C >> 2) & 0x20202020u);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                R[j][r] = s[slot_of(j, 0)];     // a0 (r = 0) / a1 (r = 1): low half
                R[j][2 + r] = s[slot_of(j, 1)]; // a2 / a3: high half
            }
        }
    }
};

template <>
struct StreamFormat<8, 128> {
    static constexpr int kSteps = 4;
    static constexpr int kWords = 16, kSets = 1, kShift = 0;
    __host__ __device__ static constexpr int set_of(int) { return 0; }
    __device__ static void pack(const uint32_t (&c)[2][8], uint32_t (&w)[kWords])
    {
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int a = 0; a < 4; ++a)
                w[j * 4 + a] = c[a & 1][2 * j + (a >> 1)];
    }
    __device__ static __forceinline__ void expand(const uint8_t *unit, int lane, uint32_t (&R)[4][4])
    {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint4 v = *reinterpret_cast<const uint4 *>(unit + j * 512 + lane * 16);
            R[j][0] = v.x;
            R[j][1] = v.y;
            R[j][2] = v.z;
            R[j][3] = v.w;
        }
    }
};

// True when no earlier MMA step of a unit feeds the accumulator set of step j.
template <typename F>
__host__ __device__ constexpr bool stream_first_in_set(int j)
{
    for (int i = 0; i < j; ++i)
        if (F::set_of(i) == F::set_of(j))
            return false;
    return true;
}

// Where lane `lane` finds word i of its kWords words inside a unit's code block: 16-byte pieces first (512 bytes per piece
// index), then one 8-byte piece, then one 4-byte piece, each lane-major -- what the formats' expand() functions read.
template <int Q, int UW>
__host__ __device__ constexpr int stream_word_offset(int lane, int i)
{
    constexpr int kWords = StreamFormat<Q, UW>::kWords;
    constexpr int n16 = kWords / 4, has8 = (kWords % 4) >= 2 ? 1 : 0;
    if (i < n16 * 4)
        return (i / 4) * 512 + lane * 16 + (i % 4) * 4;
    if (has8 && i < n16 * 4 + 2)
        return n16 * 512 + lane * 8 + (i - n16 * 4) * 4;
    return n16 * 512 + has8 * 256 + lane * 4;
}

// ---- 64-feature units (scale groups of 64): a lane owns rows g and g + 8 and 16 features; the unit has two MMA steps.
// Lane t takes its 16 features from the 32-feature run t / 2 of the unit: code(j, a, y) = the row's code at element
// 31 - 8 y - (4 (t % 2) + 2 j + (a >> 1)) of that run.  All four A registers of a step come out with the same power of two.
template <>
struct StreamFormat<2, 64> {
    static constexpr int kSteps = 2, kWords = 2, kSets = 2, kShift = 2;
    __host__ __device__ static constexpr int set_of(int j) { return j; }
    // word 0: a0, a1 of both steps; word 1: a2, a3.  Bits 0-1: (j 0, first a), 2-3: (j 1, first a), 4-5: (j 0, second a), 6-7: (j 1, second a)
    __device__ static void pack(const uint32_t (&c)[2][8], uint32_t (&w)[kWords])
    {
#pragma unroll
        for (int h = 0; h < 2; ++h)
            w[h] = c[0][h] | (c[0][2 + h] << 2) | (c[1][h] << 4) | (c[1][2 + h] << 6);
    }
    __device__ static __forceinline__ void expand(const uint8_t *unit, int lane, uint32_t (&R)[kSteps][4])
    {
        const uint2 v = *reinterpret_cast<const uint2 *>(unit + lane * 8);
        const uint32_t w[2] = { v.x, v.y };
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const uint32_t hi = w[h] >> 4;
            R[0][2 * h] = w[h] & 0x03030303u;     // row g
            R[1][2 * h] = w[h] & 0x0c0c0c0cu;
            R[0][2 * h + 1] = hi & 0x03030303u;   // row g + 8
            R[1][2 * h + 1] = hi & 0x0c0c0c0cu;
        }
    }
};

template <>
struct StreamFormat<4, 64> {
    static constexpr int kSteps = 2, kWords = 4, kSets = 2, kShift = 4;
    __host__ __device__ static constexpr int set_of(int j) { return j; }
    __device__ static void pack(const uint32_t (&c)[2][8], uint32_t (&w)[kWords])
    {
#pragma unroll
        for (int a = 0; a < 4; ++a)
            w[a] = c[a & 1][a >> 1] | (c[a & 1][2 + (a >> 1)] << 4);
    }
    __device__ static __forceinline__ void expand(const uint8_t *unit, int lane, uint32_t (&R)[kSteps][4])
    {
        const uint4 v = *reinterpret_cast<const uint4 *>(unit + lane * 16);
        const uint32_t w[4] = { v.x, v.y, v.z, v.w };
#pragma unroll
        for (int a = 0; a < 4; ++a) {
            R[0][a] = w[a] & 0x0f0f0f0fu;
            R[1][a] = w[a] & 0xf0f0f0f0u;
        }
    }
};

// three bits: the eight codes of a byte lane are the lane's (step, register) pairs; slots 0, 3, 6, 2 (times 1) hold step 0's
// registers a0..a3, slots 1, 4, 7, 5 (times 8) step 1's.  Byte layout as the 128-feature format.
template <>
struct StreamFormat<3, 64> {
    static constexpr int kSteps = 2, kWords = 3, kSets = 2, kShift = 3;
    __host__ __device__ static constexpr int set_of(int j) { return j; }
    __host__ __device__ static constexpr int slot_of(int j, int a) { return j == 0 ? (a == 0 ? 0 : a == 1 ? 3 : a == 2 ? 6 : 2) : (a == 0 ? 1 : a == 1 ? 4 : a == 2 ? 7 : 5); }
    __device__ static void pack(const uint32_t (&c)[2][8], uint32_t (&w)[kWords])
    {
        uint32_t s[8];
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int a = 0; a < 4; ++a)
                s[slot_of(j, a)] = c[a & 1][2 * j + (a >> 1)];
        w[0] = s[0] | (s[1] << 3) | ((s[2] & 0x03030303u) << 6);
        w[1] = s[3] | (s[4] << 3) | ((s[5] & 0x03030303u) << 6);
        w[2] = s[6] | (s[7] << 3) | (((s[2] >> 2) & 0x01010101u) << 6) | (((s[5] >> 2) & 0x01010101u) << 7);
    }
    __device__ static __forceinline__ void expand(const uint8_t *unit, int lane, uint32_t (&R)[kSteps][4])
    {
        const uint2 v = *reinterpret_cast<const uint2 *>(unit + lane * 8);
        const uint32_t A = v.x, B = v.y, C = *reinterpret_cast<const uint32_t *>(unit + 256 + lane * 4);
        uint32_t s[8];
        s[0] = A & 0x07070707u;
        s[1] = A & 0x38383838u;
        s[3] = B & 0x07070707u;
        s[4] = B & 0x38383838u;
        s[6] = C & 0x07070707u;
        s[7] = C & 0x38383838u;
        s[2] = ((A >> 6) & 0x03030303u) | ((C >> 4) & 0x04040404u);
        s[5] = ((B >> 3) & 0x18181818u) | ((C >> 2) & 0x20202020u);
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int a = 0; a < 4; ++a)
                R[j][a] = s[slot_of(j, a)];
    }
};

template <>
struct StreamFormat<8, 64> {
    static constexpr int kSteps = 2, kWords = 8, kSets = 1, kShift = 0;
    __host__ __device__ static constexpr int set_of(int) { return 0; }
    __device__ static void pack(const uint32_t (&c)[2][8], uint32_t (&w)[kWords])
    {
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int a = 0; a < 4; ++a)
                w[j * 4 + a] = c[a & 1][2 * j + (a >> 1)];
    }
    __device__ static __forceinline__ void expand(const uint8_t *unit, int lane, uint32_t (&R)[kSteps][4])
    {
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const uint4 v = *reinterpret_cast<const uint4 *>(unit + j * 512 + lane * 16);
            R[j][0] = v.x;
            R[j][1] = v.y;
            R[j][2] = v.z;
            R[j][3] = v.w;
        }
    }
};

// ------------------------------------------------------------------------------------------ load-time re-layout
// planes [Q][N][K/32] (+ per-group fp16 scale / u8 zero point) -> stream layout.  One thread per (tile, unit, lane).
template <int Q, int UW>
__global__ void __launch_bounds__(256) prepare_stream_kernel(const uint32_t *__restrict__ planes, const __half *__restrict__ w_scale,
                                                             const uint8_t *__restrict__ w_zero, uint8_t *__restrict__ out, int N, int K, int w_signed,
                                                             int grouped, int units_per_scale, int scale_groups)
{
    using F = StreamFormat<Q, UW>;
    const int units = K / UW, KW = K >> 5;
    const int tiles = (N + 15) >> 4;
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long long)tiles * units * 32)
        return;
    const int lane = (int)(idx & 31);
    const int u = (int)((idx >> 5) % units), r = (int)((idx >> 5) / units);
    const int g = lane >> 2, t = lane & 3;
    const int unit_bytes = Q * 2 * UW + (grouped ? 64 : 0);
    uint8_t *unit = out + ((size_t)r * units + u) * unit_bytes;
    uint32_t c[2][8];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int row = r * 16 + g + 8 * h;
        const int kw = UW == 128 ? u * 4 + t : u * 2 + (t >> 1); // the 32-feature run this lane's codes come from
        uint32_t p[Q];
#pragma unroll
        for (int b = 0; b < Q; ++b)
            p[b] = row < N ? planes[((size_t)b * N + row) * KW + kw] : 0u;
        uint32_t full[8];
        planes_to_bytes<Q>(p, w_signed != 0 && row < N, full); // two's complement -> offset codes: top plane flipped
#pragma unroll
        for (int i = 0; i < 8; ++i)
            c[h][i] = UW == 128 ? full[i] : full[(4 * (t & 1) + i) & 7]; // 64-feature units: registers 4 (t % 2) .. + 3 of the run
    }
    uint32_t w[F::kWords];
    F::pack(c, w);
#pragma unroll
    for (int i = 0; i < F::kWords; ++i)
        *reinterpret_cast<uint32_t *>(unit + stream_word_offset<Q, UW>(lane, i)) = w[i];
    if (grouped && t == 0) {
        const int zoff = w_signed ? (1 << (Q - 1)) : 0;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int row = r * 16 + g + 8 * h;
            uint32_t pk = 0;
            if (row < N) {
                const size_t si = (size_t)row * scale_groups + u / units_per_scale;
                pk = __float_as_uint(__half2float(w_scale[si])) | (uint32_t)(zoff + (w_zero ? (int)w_zero[si] : 0));
            }
            *reinterpret_cast<uint32_t *>(unit + Q * 2 * UW + (2 * g + h) * 4) = pk;
        }
    }
}

// ------------------------------------------------------------------------------------------ activation records
// Store one expanded item (token m, 32-feature run kwl of this CTA's K range; a unit is uw / 32 consecutive runs) and, from
// the first lane of each unit, the unit's code sum.
__device__ __forceinline__ void stream_store_item(uint8_t *rec_base, int *sums, int MR, int uw, int kwl, int m, const uint32_t (&r)[8], int sum, bool mine)
{
    // the runs of a unit sit in consecutive lanes (the item count per token is a multiple of the runs per unit)
    sum += __shfl_xor_sync(0xffffffffu, sum, 1);
    const int sum4 = sum + __shfl_xor_sync(0xffffffffu, sum, 2);
    if (!mine)
        return;
    if (uw == 128) {
        const int ul = kwl >> 2, t = kwl & 3;
        uint8_t *dst = rec_base + ((size_t)ul * MR + m) * 128 + t * 32;
        const int swz = (m & 1) << 4;
        *reinterpret_cast<uint4 *>(dst + swz) = make_uint4(r[0], r[1], r[2], r[3]);
        *reinterpret_cast<uint4 *>(dst + (16 ^ swz)) = make_uint4(r[4], r[5], r[6], r[7]);
        if (t == 0)
            sums[ul * MR + m] = sum4;
    } else { // 64-feature units: lanes 2 w and 2 w + 1 of the MMA quad read the two halves of run w
        const int ul = kwl >> 1, w = kwl & 1;
        uint8_t *dst = rec_base + ((size_t)ul * MR + m) * 64 + w * 32;
        *reinterpret_cast<uint4 *>(dst) = make_uint4(r[0], r[1], r[2], r[3]);
        *reinterpret_cast<uint4 *>(dst + 16) = make_uint4(r[4], r[5], r[6], r[7]);
        if (w == 0)
            sums[ul * MR + m] = sum;
    }
}

__device__ __forceinline__ int stream_code_sum(const uint32_t (&r)[8], bool x_signed)
{
    if (x_signed) {
        int sum = 0;
#pragma unroll
        for (int s = 0; s < 8; ++s)
            sum = __dp4a((int)r[s], 0x01010101, sum);
        return sum;
    }
    unsigned usum = 0;
#pragma unroll
    for (int s = 0; s < 8; ++s)
        usum = __dp4a(r[s], 0x01010101u, usum);
    return (int)usum;
}

// what the activation-record builders read of a launch
struct StreamRecArgs {
    const uint32_t *X;
    size_t x_plane_words;
    const float *x_qscale;
    int M, K, x_bits, x_signed, uw;
};

__device__ __forceinline__ void prefetch_l2(const void *p)
{
    asm volatile("prefetch.global.L2 [%0];" ::"l"(p));
}

// The build runs between "the previous kernel is complete" and the first MMA, so it is kept short: items are dealt to all
// threads of the CTA (index arithmetic by a multiply-high, no division), a thread first requests the plane words of all B
// items of a batch and then expands them (one round trip to L2 per batch, not per item), and the code is instantiated
// per activation width so that only the path taken is ever fetched.
// It is preceded, BEFORE the wait on the previous kernel, by a rehearsal (warm == true): the very same instructions run
// over the same items with the loads of activation values switched off (zeros instead), which (a) brings this code into the
// instruction cache -- a CTA's first pass through cold code costs more than the arithmetic in it -- (b) asks for the
// lines the build will read to be brought into L2, walking the page table for them, and (c) writes the zero padding
// (token rows and units beyond the real ones).  The build then overwrites the records of the real items.
template <int P, int B>
__device__ __forceinline__ void stream_records_planes(const StreamRecArgs &a, uint8_t *rec_base, int *sums, int u_first, int n_units, int n_pad, int MR, bool warm)
{
    const int wsh = a.uw == 128 ? 2 : 1; // log2 of the 32-feature runs per unit
    const int words = n_pad << wsh;
    const int items = MR * words;
    const uint32_t magic = 0xffffffffu / (uint32_t)words + 1u; // idx / words == umulhi(idx, magic) for idx * words < 2^32
    const int KW = a.K >> 5;
    for (int base = 0; base < items; base += blockDim.x * B) { // every lane of a warp takes every trip (shuffles inside)
        uint32_t pl[B][P];
        int mm[B], kk[B];
        bool live[B];
#pragma unroll
        for (int i = 0; i < B; ++i) {
            const int idx = base + i * (int)blockDim.x + (int)threadIdx.x;
            mm[i] = (int)__umulhi((uint32_t)idx, magic);
            kk[i] = idx - mm[i] * words;
            live[i] = idx < items && mm[i] < a.M && (kk[i] >> wsh) < n_units;
            const uint32_t *src = a.X + (size_t)mm[i] * KW + (u_first << wsh) + kk[i];
            if (warm && live[i] && (kk[i] & 31) == 0) { // one request per 128-byte line of every plane row
#pragma unroll
                for (int b = 0; b < P; ++b)
                    prefetch_l2(src + b * a.x_plane_words);
            }
#pragma unroll
            for (int b = 0; b < P; ++b)
                pl[i][b] = (live[i] && !warm) ? __ldg(src + b * a.x_plane_words) : 0u;
        }
#pragma unroll
        for (int i = 0; i < B; ++i) {
            const int idx = base + i * (int)blockDim.x + (int)threadIdx.x;
            uint32_t r[8];
            x_bytes<P>(pl[i], a.x_signed != 0, r); // (zeros in, zeros out: no branch around the arithmetic)
            const int sum = stream_code_sum(r, a.x_signed != 0);
            stream_store_item(rec_base, sums, MR, a.uw, kk[i], mm[i], r, sum, warm ? idx < items : live[i]);
        }
    }
}

__device__ __forceinline__ void stream_records_half(const StreamRecArgs &a, uint8_t *rec_base, int *sums, int u_first, int n_units, int n_pad, int MR, bool warm)
{
    const int wsh = a.uw == 128 ? 2 : 1;
    const int words = n_pad << wsh;
    const int items = MR * words;
    const uint32_t magic = 0xffffffffu / (uint32_t)words + 1u;
    if (warm && threadIdx.x == 0)
        prefetch_l2(a.x_qscale);
    const __half hscale = warm ? __half() : __float2half(__ldg(a.x_qscale));
    for (int base = 0; base < items; base += blockDim.x) {
        const int idx = base + (int)threadIdx.x;
        const int m = (int)__umulhi((uint32_t)idx, magic), kwl = idx - m * words;
        const bool live = idx < items && m < a.M && (kwl >> wsh) < n_units;
        const uint4 *src = reinterpret_cast<const uint4 *>(reinterpret_cast<const __half *>(a.X) + (size_t)m * a.K + (size_t)((u_first << wsh) + kwl) * 32);
        uint32_t r[8];
#pragma unroll
        for (int s = 0; s < 8; ++s)
            r[s] = 0;
        if (warm && live && (kwl & 1) == 0)
            prefetch_l2(src); // 64 bytes per item: one request per 128-byte line
        if (live && !warm)
            x_bytes_from_half(src, hscale, a.x_bits, r);
        const int sum = stream_code_sum(r, true);
        stream_store_item(rec_base, sums, MR, a.uw, kwl, m, r, sum, warm ? idx < items : live);
    }
}

// Records of units [u_first, u_first + n_units) of this CTA's K range, zero-padded to n_pad units and MR token rows:
// rec[(ul * MR + m) * 128 + t * 32 + {0, 16} ^ ((m & 1) << 4)] = the lane-t halves (registers 0..3 and 4..7 of x_bytes)
// of token m, and sums[ul * MR + m] = the sum of its 128 codes (64-feature units: see stream_store_item).
// warm: the rehearsal before the dependency wait (see above).  One copy of this code per compile unit.
static __device__ __noinline__ void stream_build_records(const uint32_t *X, size_t x_plane_words, const float *x_qscale, int M, int K, int x_bits,
                                                         int x_signed, int uw, uint8_t *rec_base, int *sums, int u_first, int n_units, int n_pad,
                                                         int MR, bool warm)
{
    // (scalars, not a reference to the kernel's parameter block: a reference handed to a function that is not inlined would
    // make every thread copy the whole block to its stack first)
    const StreamRecArgs a = { X, x_plane_words, x_qscale, M, K, x_bits, x_signed, uw };
    if (a.x_qscale) {
        stream_records_half(a, rec_base, sums, u_first, n_units, n_pad, MR, warm);
        return;
    }
    const bool one = MR * n_pad * (a.uw / 32) <= (int)blockDim.x; // one item per thread at most: no batching needed
#define ABQ_RECORDS_CASE(P)                                                                                      \
    case P:                                                                                                      \
        if (one)                                                                                                 \
            stream_records_planes<P, 1>(a, rec_base, sums, u_first, n_units, n_pad, MR, warm);                   \
        else                                                                                                     \
            stream_records_planes<P, 4>(a, rec_base, sums, u_first, n_units, n_pad, MR, warm);                   \
        break;
    switch (a.x_bits) {
        ABQ_RECORDS_CASE(1)
        ABQ_RECORDS_CASE(2)
        ABQ_RECORDS_CASE(3)
        ABQ_RECORDS_CASE(4)
        ABQ_RECORDS_CASE(5)
        ABQ_RECORDS_CASE(6)
        ABQ_RECORDS_CASE(7)
    default:
        if (one)
            stream_records_planes<8, 1>(a, rec_base, sums, u_first, n_units, n_pad, MR, warm);
        else
            stream_records_planes<8, 4>(a, rec_base, sums, u_first, n_units, n_pad, MR, warm);
    }
#undef ABQ_RECORDS_CASE
}

// D(16x8, s32) = A(16x32, u8) * B(32x8, s8) + 0: first step of an accumulation (saves clearing the accumulators)
__device__ __forceinline__ void mma_u8s8_first(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1)
{
    const int z = 0;
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};\n"
                 : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(z));
}

// Shared-memory carve-up, the same arithmetic on the host (planner) and in the kernel.
struct StreamSmem {
    size_t ring, rec, sums, zero, red, bars, total;
};
__host__ __device__ inline StreamSmem stream_smem_layout(int nw, int ring, int cu, int unit_bytes, int units_pad, int MR, int tiles_per_cta, int MT, int uw)
{
    StreamSmem L;
    size_t at = 0;
    L.ring = at;
    at += (size_t)nw * ring * cu * unit_bytes;
    L.rec = at;
    at += (size_t)units_pad * MR * uw;
    L.sums = at;
    at += ((size_t)units_pad * MR * 4 + 15) & ~(size_t)15;
    L.zero = at;
    at += 32;
    L.red = at;
    at += (size_t)(nw + tiles_per_cta) * MT * 512; // [pair][token tile][16 rows][8 columns] 32-bit
    L.bars = at;
    at += (size_t)nw * kStreamMaxRing * 8;
    L.total = at + 128; // slack for aligning the base to 128 bytes
    return L;
}

// Q: weight bits.  MT: token tiles of 8 (2 for 9..16 tokens, 4 for 17..32: at most eight warps then, so that a thread may
// use up to 255 registers).  MP: token rows per column block (1, 2, 4, 8).
// GS = 8 / MP units share one set of accumulators (GROUPED only).  GROUPED: per-group scale / zero point in the stream.
template <int Q, int MT, int MP, bool GROUPED, int UW>
__global__ void __launch_bounds__(MT == 4 ? 256 : kStreamMaxWarps * 32, 1) stream_kernel(const StreamArgs a)
{
    using F = StreamFormat<Q, UW>;
    constexpr int kCodeBytes = Q * 2 * UW; // of a unit; its 64 parameter bytes follow
    static_assert(GROUPED || UW == 128, "64-feature units exist for scale groups of 64 only");
    constexpr int GS = GROUPED ? 8 / MP : 1;
    constexpr int MR = MT >= 2 ? 8 * MT : MP; // token rows of a record
    static_assert(MT == 1 || MP == 8, "several token tiles only with full column blocks");
    static_assert(MT == 1 || MT == 2 || MT == 4, "8, 16 or 32 token rows per launch");
    extern __shared__ __align__(128) uint8_t smem_raw[];
    uint8_t *smem = smem_raw + ((128u - (smem_u32(smem_raw) & 127u)) & 127u);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int nw = a.nw;
    // (without a K split, which is the common case, a CTA's position is its block index)
    const int s = a.slices > 1 ? blockIdx.x / a.ctas_per_slice : 0;
    const int cb = blockIdx.x - s * a.ctas_per_slice;
    // tiles [r_begin, r_end) of this CTA: an even share, the first tiles_r CTAs of the slice taking one more
    const int r_begin = cb * a.tiles_q + min(cb, a.tiles_r);
    const int T = a.tiles_q + (cb < a.tiles_r ? 1 : 0);
    const int r_end = r_begin + T;
    const int max_T = a.max_tiles;
    const int u0 = s * a.units_per_slice;                        // first unit of this CTA's K range
    const int n_units = max(0, min(a.units - u0, a.units_per_slice)); // its unit count
    const int units_pad = a.units_per_slice;                     // records are padded to whole chunks
    const int cpt = n_units == a.units_per_slice ? a.cpt_full : (n_units + a.cu - 1) / a.cu; // chunks per tile
    const int total_chunks = T * cpt;
    const int chunk_bytes = a.cu * a.unit_bytes;

    const StreamSmem L = stream_smem_layout(nw, a.ring, a.cu, a.unit_bytes, units_pad, MR, max_T, MT, UW);
    uint8_t *ring_base = smem + L.ring;
    uint8_t *rec_base = smem + L.rec;
    int *sums = reinterpret_cast<int *>(smem + L.sums);
    const uint8_t *zero_base = smem + L.zero;
    int *red = reinterpret_cast<int *>(smem + L.red);
    uint64_t *full = reinterpret_cast<uint64_t *>(smem + L.bars) + warp * kStreamMaxRing;

    if (lane == 0) {
        for (int i = 0; i < a.ring; ++i)
            mbar_init(&full[i], 1);
        fence_mbar_init();
    }
    if (threadIdx.x < 8)
        reinterpret_cast<uint32_t *>(smem + L.zero)[threadIdx.x] = 0;
    __syncwarp();
    pdl_launch_dependents();

    // ---- this warp's chunks: [c_begin, c_end) of the CTA's T * cpt chunks (tile-major)
    __shared__ int chunk_bound[kStreamMaxWarps + 1];
    // (the same share for every warp, the first warps served first: the warps that hold a share of a tile are then consecutive)
    const int chunks_per_warp = (total_chunks + nw - 1) >> a.nw_shift;
    if ((int)threadIdx.x <= nw)
        chunk_bound[threadIdx.x] = min((int)threadIdx.x * chunks_per_warp, total_chunks); // read again after the barriers below
    const int c_begin = min(warp * chunks_per_warp, total_chunks);
    const int c_end = min((warp + 1) * chunks_per_warp, total_chunks);
    uint8_t *my_ring = ring_base + (size_t)warp * a.ring * chunk_bytes;

    // request side (lane 0): cursor over the chunks in consumption order
    int q_cit = 0, q_left = 0;
    const uint8_t *q_src = a.Wp; // where the next chunk starts: chunks of a tile follow one another in memory
    if (cpt > 0) {
        const int q_tile = cpt == 1 ? c_begin : cpt == a.cpt_full ? (int)__umulhi((uint32_t)c_begin, a.cpt_magic) : c_begin / cpt; // (no magic for 1)
        q_cit = c_begin - q_tile * cpt;
        q_left = c_end - c_begin;
        q_src = a.Wp + ((size_t)(r_begin + q_tile) * a.units + u0 + (size_t)q_cit * a.cu) * a.unit_bytes;
    }
    const uint32_t last_chunk_bytes = (uint32_t)(n_units - (cpt - 1) * a.cu) * a.unit_bytes;        // of a tile's K range
    const size_t tile_gap = (size_t)(a.units - n_units) * a.unit_bytes;                               // K range of the other slices
    // (common case: every chunk has all its units and the tiles of this CTA follow one another in memory, so the requests
    // are equal pieces of one contiguous byte range and need no bookkeeping)
    const bool uniform_chunks = last_chunk_bytes == (uint32_t)chunk_bytes && tile_gap == 0;
    auto issue = [&](int slot) {
        if (uniform_chunks) {
            mbar_arrive_expect_tx(&full[slot], (uint32_t)chunk_bytes);
            bulk_load(my_ring + (size_t)slot * chunk_bytes, q_src, (uint32_t)chunk_bytes, &full[slot]);
            q_src += chunk_bytes;
            --q_left;
            return;
        }
        const bool last = q_cit == cpt - 1;
        const uint32_t bytes = last ? last_chunk_bytes : (uint32_t)chunk_bytes;
        mbar_arrive_expect_tx(&full[slot], bytes);
        bulk_load(my_ring + (size_t)slot * chunk_bytes, q_src, bytes, &full[slot]);
        q_src += bytes + (last ? tile_gap : 0);
        q_cit = last ? 0 : q_cit + 1;
        --q_left;
    };
    if (lane == 0) {
        for (int slot = 0; slot < a.prefill && q_left > 0; ++slot)
            issue(slot); // weights never depend on an earlier kernel: request them before the dependency wait
    }

    // ---- everything that does not depend on the previous kernel happens before the wait on it, where it costs nothing:
    // which warps hold a share of which tile (for the final reduction), and which output this thread finishes first
    __shared__ unsigned short tile_warps[64]; // [tile of this CTA] -> first warp | (last warp + 1) << 8
    __syncthreads();                          // chunk_bound is written
    for (int tl = threadIdx.x; tl < T && tl < 64; tl += blockDim.x) {
        const int lo = tl * cpt, hi = lo + cpt;
        int w_lo = nw, w_hi = 0;
        for (int w = 0; w < nw; ++w) {
            if (chunk_bound[w] < chunk_bound[w + 1] && chunk_bound[w] < hi && chunk_bound[w + 1] > lo) {
                w_lo = min(w_lo, w);
                w_hi = w + 1;
            }
        }
        tile_warps[tl] = (unsigned short)(min(w_lo, w_hi) | (w_hi << 8));
    }
    const int per_tile = a.M * 16; // outputs of a tile; output idx of the CTA is tile idx / per_tile, token (idx % per_tile) / 16, row idx % 16
    const int first_tl = (int)__umulhi(threadIdx.x, a.per_tile_magic), first_i = (int)threadIdx.x - first_tl * per_tile;
    // The activation records.  Common case (plane input of 8 or 4 bits, at most kFast items per thread): everything about
    // a thread's items that can be known now is computed now -- where the plane words come from, where the record goes --
    // so that after the wait only loads, the bit shuffle and stores remain, in straight-line code.  Other cases run the
    // general routine, rehearsed here with the loads switched off.  Either way: the records' zero padding is written, the
    // lines to be read (and the lines this CTA will store its results to) are requested into L2, page-table walk included.
    constexpr int kFast = 4;
    const int rec_words = units_pad * (UW / 32), rec_items = MR * rec_words;
    const int rec_batches = (rec_items + (int)blockDim.x - 1) >> (a.nw_shift + 5); // (the CTA has 32 << nw_shift threads)
    const bool rec_fast = !a.x_qscale && (a.x_bits == 8 || a.x_bits == 4) && rec_batches <= kFast;
    const uint32_t *it_src[kFast]; // plane 0 word of the item, or null: padding (already zero)
    uint32_t it_dst[kFast];        // byte offset of the record from rec_base | 1: this lane also stores the unit's code sum
    if (rec_fast) {
        const uint32_t magic = a.rec_magic; // idx / rec_words == umulhi(idx, magic) here
#pragma unroll
        for (int i = 0; i < kFast; ++i) {
            it_src[i] = nullptr;
            it_dst[i] = 0;
            if (i >= rec_batches) // (the same for every thread: one token needs one batch)
                continue;
            const int idx = i * (int)blockDim.x + (int)threadIdx.x;
            const int m = (int)__umulhi((uint32_t)idx, magic), kwl = idx - m * rec_words;
            const bool live = idx < rec_items && m < a.M && kwl / (UW / 32) < n_units;
            it_src[i] = live ? a.X + (size_t)m * (a.K >> 5) + (size_t)u0 * (UW / 32) + kwl : nullptr;
            const int ul = kwl / (UW / 32), part = kwl % (UW / 32);
            it_dst[i] = (uint32_t)(((size_t)ul * MR + m) * UW + part * 32) | (part == 0 ? 1u : 0u) | ((uint32_t)(m & 1) << 1);
            if (live && (kwl & 31) == 0)
                for (int b = 0; b < a.x_bits; ++b)
                    prefetch_l2(it_src[i] + b * a.x_plane_words);
        }
        // zero padding: the whole record area (real items are overwritten after the wait)
        for (int i = threadIdx.x; i < (int)((size_t)units_pad * MR * UW / 16); i += blockDim.x)
            reinterpret_cast<uint4 *>(rec_base)[i] = make_uint4(0, 0, 0, 0);
        for (int i = threadIdx.x; i < units_pad * MR; i += blockDim.x)
            sums[i] = 0;
    } else {
        stream_build_records(a.X, a.x_plane_words, a.x_qscale, a.M, a.K, a.x_bits, a.x_signed, a.uw, rec_base, sums, u0, n_units, units_pad, MR, true);
    }
    {
        const size_t esz = a.out_dtype == ABQ_OUT_INT32 ? 4 : 2;
        for (int i = threadIdx.x; i < a.M; i += blockDim.x)
            prefetch_l2(reinterpret_cast<const uint8_t *>(a.D) + ((size_t)i * a.N + (size_t)r_begin * 16) * esz);
    }
    // ---- activations: everything below may depend on the kernel launched just before
    pdl_wait_prior_grid();
    if (lane == 0) {
        for (int slot = a.prefill; slot < a.ring && q_left > 0; ++slot)
            issue(slot);
    }
    __shared__ uint32_t ar_epoch;
    if (a.ar.world > 1 && threadIdx.x == 0) // (only the last CTA of a launch advances the counter, after all have read it)
        ar_epoch = *reinterpret_cast<volatile uint32_t *>(a.ar.counter) + 1u;
    if (rec_fast) {
        auto build = [&](auto width_tag) {
            constexpr int P = decltype(width_tag)::value;
            uint32_t pl[kFast][P];
#pragma unroll
            for (int i = 0; i < kFast; ++i) {
                if (i < rec_batches) { // (uniform: no predicated loads for batches that do not exist)
#pragma unroll
                    for (int b = 0; b < P; ++b)
                        pl[i][b] = it_src[i] ? __ldg(it_src[i] + b * a.x_plane_words) : 0u;
                }
            }
#pragma unroll
            for (int i = 0; i < kFast; ++i) {
                if (i < rec_batches) { // the same for every thread of the CTA: the shuffles below see whole warps
                    uint32_t r[8];
                    x_bytes<P>(pl[i], a.x_signed != 0, r);
                    int sum = stream_code_sum(r, a.x_signed != 0);
                    sum += __shfl_xor_sync(0xffffffffu, sum, 1); // the runs of a unit sit in consecutive lanes
                    if (UW == 128)
                        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
                    if (it_src[i]) {
                        uint8_t *dst = rec_base + (it_dst[i] & ~3u);
                        const int swz = UW == 128 ? (int)(it_dst[i] & 2u) << 3 : 0; // odd token rows swap their 16-byte halves
                        *reinterpret_cast<uint4 *>(dst + swz) = make_uint4(r[0], r[1], r[2], r[3]);
                        *reinterpret_cast<uint4 *>(dst + (16 ^ swz)) = make_uint4(r[4], r[5], r[6], r[7]);
                        if (it_dst[i] & 1u)
                            sums[(it_dst[i] & ~3u) / UW] = sum;
                    }
                }
            }
        };
        if (a.x_bits == 8)
            build(std::integral_constant<int, 8>{});
        else
            build(std::integral_constant<int, 4>{});
    } else {
        stream_build_records(a.X, a.x_plane_words, a.x_qscale, a.M, a.K, a.x_bits, a.x_signed, a.uw, rec_base, sums, u0, n_units, units_pad, MR, false);
    }
    __syncthreads();

    // lane constants of the B fragment fetch: column c = g holds token (g % MP) of unit (g / MP) of a block
    const int my_m = g & (MP - 1);
    const int my_slot = GS > 1 ? g / MP : 0;
    const int rec_lane = UW == 128 ? my_m * 128 + t * 32 : my_m * 64 + t * 16;
    const int swz = (my_m & 1) << 4;
    const int zoff = a.w_signed ? (1 << (Q - 1)) : 0;

    bool ok = true;
    int slot = 0;
    uint32_t phase = 0;
    // tile (local) and chunk within it of the chunk being consumed
    int tile_l = cpt > 1 ? (cpt == a.cpt_full ? (int)__umulhi((uint32_t)c_begin, a.cpt_magic) : c_begin / cpt) : c_begin;
    int cit = cpt > 0 ? c_begin - tile_l * cpt : 0;

    int acc_run[F::kSets][MT][4]; // without per-group scales: integer sums over the whole K range of a tile
    float facc[MT][4];
    int xs[MT][2];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
#pragma unroll
            for (int k = 0; k < F::kSets; ++k)
                acc_run[k][mt][e] = 0;
            facc[mt][e] = 0.f;
        }
        xs[mt][0] = xs[mt][1] = 0;
    }

    // |acc0 + acc1 / 2^kShift - (zero + offset) * sum(x)| of one 128-feature group stays below 2^22 for the narrow widths:
    // int -> float by the 1.5 * 2^23 trick (two plain ALU/FMA operations) instead of a conversion instruction
    constexpr long long kBound = (long long)UW * 128 * (((1 << Q) - 1) + ((1 << Q) - 1) + (1 << (Q - 1)));
    constexpr bool kMagic = kBound < (1LL << 22);

    for (int ci = c_begin; ci < c_end && ok; ++ci) {
        ok = mbar_wait_bounded(&full[slot], phase, a.status, STATUS_TIMEOUT_TMA);
        if (!ok)
            break;
        const uint8_t *stage = my_ring + (size_t)slot * chunk_bytes;
        const int uf = cit * a.cu;              // first unit of the chunk within this CTA's K range
        const int nu = min(a.cu, n_units - uf); // units in the chunk
        // The loops over blocks and over the units of a block stay rolled (two units per trip): a warp only sees a few dozen
        // units per launch, and straight-line code that long is fetched from the instruction cache about as often as it
        // is executed -- measured, instruction fetch and not arithmetic was what this loop waited for when it was unrolled.
#pragma unroll 1
        for (int ub = 0; ub < nu; ub += GS) {
            const uint8_t *blk = stage + (size_t)ub * a.unit_bytes;
            const int left = nu - ub; // units of this block that exist
            // GROUPED: the block's own accumulators; blocks of several units keep two sets, for even and odd units, so that a
            // unit's MMAs do not queue behind those of the unit before it
            constexpr int kPar = GROUPED && GS >= 2 ? 2 : 1;
            int acc_block[kPar][F::kSets][MT][4];
            if (GROUPED && GS >= 2) {
#pragma unroll
                for (int i = 0; i < kPar * F::kSets * MT * 4; ++i)
                    (&acc_block[0][0][0][0])[i] = 0;
            }
            auto run_unit = [&](int ui, auto par_tag) { // ui: unit of the block; par_tag: which accumulator set (compile time)
                constexpr int kP = decltype(par_tag)::value;
                const uint8_t *unit = blk + ui * a.unit_bytes;
                uint32_t R[F::kSteps][4];
                F::expand(unit, lane, R);
                const uint8_t *rec = rec_base + (size_t)(uf + ub + ui) * MR * UW;
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    const uint8_t *bp = (GS == 1 || my_slot == ui) ? rec + mt * 8 * UW + rec_lane : zero_base;
                    uint32_t bf[2 * F::kSteps];
                    if (UW == 128) {
                        const uint4 blo = *reinterpret_cast<const uint4 *>(bp + swz);
                        const uint4 bhi = *reinterpret_cast<const uint4 *>(bp + (16 ^ swz));
                        bf[0] = blo.x, bf[1] = blo.y, bf[2] = blo.z, bf[3] = blo.w;
                        bf[4 % (2 * F::kSteps)] = bhi.x, bf[5 % (2 * F::kSteps)] = bhi.y, bf[6 % (2 * F::kSteps)] = bhi.z, bf[7 % (2 * F::kSteps)] = bhi.w;
                    } else {
                        const uint4 bq = *reinterpret_cast<const uint4 *>(bp);
                        bf[0] = bq.x, bf[1] = bq.y, bf[2] = bq.z, bf[3] = bq.w;
                    }
#pragma unroll
                    for (int j = 0; j < F::kSteps; ++j) {
                        int(&acc)[4] = GROUPED ? acc_block[kP][F::set_of(j)][mt] : acc_run[F::set_of(j)][mt];
                        // a single-unit block starts its sets from zero with the MMA itself
                        if (GROUPED && GS == 1 && stream_first_in_set<F>(j))
                            mma_u8s8_first(acc, R[j][0], R[j][1], R[j][2], R[j][3], bf[2 * j], bf[2 * j + 1]);
                        else
                            mma_u8<false>(acc, R[j][0], R[j][1], R[j][2], R[j][3], bf[2 * j], bf[2 * j + 1]);
                    }
                }
                if (!GROUPED) {
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt) {
                        if (MP == 1) { // one token: every column is that token
                            const int sv = sums[uf + ub + ui];
                            xs[mt][0] += sv;
                            xs[mt][1] += sv;
                        } else {       // columns 2 t, 2 t + 1 are tokens (2 t) % MP, + 1 (columns beyond MP repeat tokens and are ignored)
                            const int2 sv = *reinterpret_cast<const int2 *>(sums + (uf + ub + ui) * MR + 8 * mt + ((2 * t) & (MP - 1)));
                            xs[mt][0] += sv.x;
                            xs[mt][1] += sv.y;
                        }
                    }
                }
            };
            if (GS == 1) {
                run_unit(0, std::integral_constant<int, 0>{});
            } else {
#pragma unroll 1
                for (int ui = 0; ui < GS && ui < left; ui += 2) {
                    run_unit(ui, std::integral_constant<int, 0>{});
                    if (ui + 1 < left)
                        run_unit(ui + 1, std::integral_constant<int, kPar - 1>{});
                }
            }
            if (GROUPED) {
                // fold the block: column 2 t + j of the accumulators is token (col % MP) of unit ub + col / MP
                const int ul = uf + ub; // first unit of the block within the CTA's K range (a multiple of GS)
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    uint2 pk[2]; // [column of the pair] -> (row g, row g + 8)
                    int xv[2];
                    if (MP == 1) {
                        pk[0] = (2 * t < left) ? *reinterpret_cast<const uint2 *>(blk + (2 * t) * a.unit_bytes + kCodeBytes + 8 * g) : make_uint2(0, 0);
                        pk[1] = (2 * t + 1 < left) ? *reinterpret_cast<const uint2 *>(blk + (2 * t + 1) * a.unit_bytes + kCodeBytes + 8 * g) : make_uint2(0, 0);
                        const int2 sv = *reinterpret_cast<const int2 *>(sums + ul + 2 * t);
                        xv[0] = sv.x;
                        xv[1] = sv.y;
                    } else {
                        const int sl = (2 * t) / MP; // both columns of the pair belong to the same unit
                        pk[0] = (GS == 1 || sl < left) ? *reinterpret_cast<const uint2 *>(blk + sl * a.unit_bytes + kCodeBytes + 8 * g) : make_uint2(0, 0);
                        pk[1] = pk[0];
                        const int2 sv = *reinterpret_cast<const int2 *>(sums + (ul + sl) * MR + 8 * mt + ((2 * t) & (MP - 1)));
                        xv[0] = sv.x;
                        xv[1] = sv.y;
                    }
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const uint32_t p = (e >> 1) ? pk[e & 1].y : pk[e & 1].x;
                        const float sc_w = __uint_as_float(p & ~kZeroMask);
                        const int z = (int)(p & kZeroMask);
                        int v = acc_block[0][0][mt][e];
                        if (kPar == 2)
                            v += acc_block[kPar - 1][0][mt][e];
                        if (F::kSets == 2) { // exact: every term of that set is a multiple of 2^kShift
                            int hi = acc_block[0][F::kSets - 1][mt][e];
                            if (kPar == 2)
                                hi += acc_block[kPar - 1][F::kSets - 1][mt][e];
                            v += hi >> F::kShift;
                        }
                        v -= z * xv[e & 1];
                        const float fv = kMagic ? __int_as_float(v + 0x4b400000) - 12582912.0f : (float)v;
                        facc[mt][e] = fmaf(fv, sc_w, facc[mt][e]);
                    }
                }
            }
        }
        __syncwarp();
        if (lane == 0 && q_left > 0)
            issue(slot); // the slot just consumed is free again
        if (++slot == a.ring) {
            slot = 0;
            phase ^= 1;
        }
        // ---- end of this warp's share of a tile: hand the partial sums over
        const bool tile_done = cit == cpt - 1 || ci == c_end - 1;
        if (tile_done) {
            int *dst = red + (size_t)(warp + tile_l) * MT * 128; // [token tile][16 rows][8 columns]
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                int v[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    if (GROUPED) {
                        v[e] = __float_as_int(facc[mt][e]);
                        facc[mt][e] = 0.f;
                    } else {
                        int z = zoff;
                        const int n = (r_begin + tile_l) * 16 + g + 8 * (e >> 1);
                        if (a.scale_mode == ABQ_SCALE_CHANNEL && a.w_zero && n < a.N)
                            z += a.w_zero[n];
                        int x = acc_run[0][mt][e];
                        if (F::kSets == 2)
                            x += acc_run[F::kSets - 1][mt][e] >> F::kShift;
                        v[e] = x - z * xs[mt][e & 1];
#pragma unroll
                        for (int k = 0; k < F::kSets; ++k)
                            acc_run[k][mt][e] = 0;
                    }
                }
                xs[mt][0] = xs[mt][1] = 0;
                if (GS > 1) {
                    // columns c and c' with c % MP == c' % MP are the same token seen through different units: add them here,
                    // in the warp, so that the tile's partial is [16 rows][MP tokens] (columns 0 .. MP - 1)
                    float f[4] = { __int_as_float(v[0]), __int_as_float(v[1]), __int_as_float(v[2]), __int_as_float(v[3]) };
                    if (MP == 1) {
                        f[0] += f[1];
                        f[2] += f[3];
                    }
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        if (MP <= 2)
                            f[e] += __shfl_xor_sync(0xffffffffu, f[e], 1);
                        f[e] += __shfl_xor_sync(0xffffffffu, f[e], 2);
                        v[e] = __float_as_int(f[e]);
                    }
                }
                if (GS == 1 || 2 * t < MP || t == 0) {
                    *reinterpret_cast<int2 *>(dst + mt * 128 + g * 8 + 2 * t) = make_int2(v[0], v[1]);
                    *reinterpret_cast<int2 *>(dst + mt * 128 + (g + 8) * 8 + 2 * t) = make_int2(v[2], v[3]);
                }
            }
        }
        if (++cit == cpt) {
            cit = 0;
            ++tile_l;
        }
    }
    // A wait that expired may have left copies in flight: give them one more bounded chance to land before the shared
    // memory they target is released.
    if (!ok && lane == 0) {
        for (int i = 0; i < a.ring; ++i)
            mbar_wait_bounded(&full[i], 0, nullptr, 0);
    }
    __syncthreads();

    // ---- the CTA's tiles: add the warps' partial sums in warp order, finish, store.  Thread per (tile, token, row).
    auto tile_sum = [&](int tl, int m, int row) -> int {
        int isum = 0;
        float fsum = 0.f;
        const int w_lo = tile_warps[tl] & 0xff, w_hi = tile_warps[tl] >> 8; // the warps that hold a share of this tile
        for (int w = w_lo; w < w_hi; ++w) {
            const int v = red[(size_t)(w + tl) * MT * 128 + (m >> 3) * 128 + row * 8 + (m & 7)];
            if (GROUPED)
                fsum += __int_as_float(v);
            else
                isum += v;
        }
        return GROUPED ? __float_as_int(fsum) : isum;
    };
    auto finish = [&](int r, int m, int row, int v) {
        const int n = r * 16 + row;
        if (n >= a.N)
            return;
        const size_t o = (size_t)m * a.N + n;
        if (a.out_dtype == ABQ_OUT_INT32) {
            reinterpret_cast<int *>(a.D)[o] = v;
        } else {
            __half h;
            if (a.scale_mode == ABQ_SCALE_TENSOR_COMPAT) {
                h = __hmul(__int2half_rn(v), ld_half(a.C));
            } else {
                float f = GROUPED ? __int_as_float(v) : (float)v * __half2float(ld_half(a.w_scale + n));
                if (a.x_scale)
                    f *= a.x_scale[m];
                h = __float2half_rn(f);
            }
            if (a.residual)
                h = __hadd(h, a.residual[o]);
            reinterpret_cast<__half *>(a.D)[o] = h;
        }
    };
    if (a.slices == 1 && a.ar.world > 1) {
        // ---- all-reduce over the ranks, fused: push this CTA's partial tiles to every rank, flag them, wait for the
        // other ranks' flags of the same tiles, add what they pushed (rank order, fp32).
        const uint32_t epoch = ar_epoch;
        const int W = a.ar.world, par = (int)(epoch & 1u);
        auto half_of = [&](int r, int m, int row, int v) -> __half {
            const int n = r * 16 + row;
            float f = GROUPED ? __int_as_float(v) : (float)v * (n < a.N ? __half2float(ld_half(a.w_scale + n)) : 0.f);
            if (a.x_scale)
                f *= a.x_scale[m];
            return __float2half_rn(f);
        };
        for (int idx = threadIdx.x; idx < T * per_tile; idx += blockDim.x) {
            const int tl = idx == (int)threadIdx.x ? first_tl : idx / per_tile, i = idx == (int)threadIdx.x ? first_i : idx - tl * per_tile;
            const int m = i >> 4, row = i & 15, n = (r_begin + tl) * 16 + row;
            if (n < a.N) {
                const __half h = half_of(r_begin + tl, m, row, tile_sum(tl, m, row));
                const size_t at = ((size_t)(par * W + a.ar.rank) * a.ar.rows_cap + a.ar.row0 + m) * a.N + n;
                for (int p = 0; p < W; ++p)
                    a.ar.recv[p][at] = h; // 16 consecutive threads write the 32 bytes of a token row of the tile
            }
        }
        __threadfence_system(); // this thread's pushes are visible system-wide before ...
        __syncthreads();        // ... any flag of this CTA goes out
        bool arrived = true;
        for (int i = threadIdx.x; i < W * T; i += blockDim.x) {
            const int p = i / T, tl = i - p * T;
            if (p == a.ar.rank)
                continue;
            uint32_t *theirs = a.ar.flags[p] + (size_t)(par * W + a.ar.rank) * a.tiles + r_begin + tl;
            asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(theirs), "r"(epoch) : "memory");
            const uint32_t *mine = a.ar.flags[a.ar.rank] + (size_t)(par * W + p) * a.tiles + r_begin + tl;
            const unsigned long long t0 = globaltimer_ns();
            for (;;) {
                uint32_t v;
                asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
                if (v == epoch)
                    break;
                if (globaltimer_ns() - t0 > kWaitLimitNs) { // the peer never arrived: record it and carry on (the sum is then void)
                    if (a.status)
                        atomicOr(a.status, STATUS_TIMEOUT_PIPE);
                    arrived = false;
                    break;
                }
            }
        }
        (void)arrived;
        __syncthreads();
        for (int idx = threadIdx.x; idx < T * per_tile; idx += blockDim.x) {
            const int tl = idx / per_tile, i = idx - tl * per_tile;
            const int m = i >> 4, row = i & 15, n = (r_begin + tl) * 16 + row;
            if (n >= a.N)
                continue;
            float f = 0.f;
            for (int p = 0; p < W; ++p) {
                const size_t at = ((size_t)(par * W + p) * a.ar.rows_cap + a.ar.row0 + m) * a.N + n;
                // written by another GPU into this one's memory: read past the L1 (no stale line)
                f += __half2float(__ushort_as_half(__ldcv(reinterpret_cast<const unsigned short *>(a.ar.recv[a.ar.rank] + at))));
            }
            __half h = __float2half_rn(f);
            if (a.residual)
                h = __hadd(h, a.residual[(size_t)m * a.N + n]);
            reinterpret_cast<__half *>(a.D)[(size_t)m * a.N + n] = h;
        }
        __syncthreads();
        if (threadIdx.x == 0) { // the last CTA of the launch advances the call counter
            const uint32_t done = atomicAdd(a.ar.counter + 1, 1u);
            if (done == gridDim.x - 1) {
                a.ar.counter[1] = 0;
                __threadfence();
                a.ar.counter[0] = epoch;
            }
        }
        return;
    }
    if (a.slices == 1) {
        for (int idx = threadIdx.x; idx < T * per_tile; idx += blockDim.x) { // all threads busy, whatever the token count
            const int tl = idx == (int)threadIdx.x ? first_tl : idx / per_tile, i = idx == (int)threadIdx.x ? first_i : idx - tl * per_tile;
            finish(r_begin + tl, i >> 4, i & 15, tile_sum(tl, i >> 4, i & 15));
        }
        return;
    }
    // ---- K split over CTAs as well: a workspace slot per slice, the CTA arriving last at a tile's counter adds the
    // slots in slice order (the result does not depend on who finishes)
    for (int idx = threadIdx.x; idx < T * per_tile; idx += blockDim.x) {
        const int tl = idx / per_tile, i = idx - tl * per_tile;
        a.partials[((size_t)s * a.tiles + r_begin + tl) * (size_t)per_tile + i] = tile_sum(tl, i >> 4, i & 15);
    }
    __threadfence();
    __syncthreads();
    int *last = red; // reuse: one flag per tile of this CTA
    for (int tl = threadIdx.x; tl < T; tl += blockDim.x) {
        const int old = atomicAdd(a.counters + r_begin + tl, 1);
        last[tl] = old == a.slices - 1;
        if (old == a.slices - 1)
            a.counters[r_begin + tl] = 0; // leave the counter ready for the next launch
    }
    __syncthreads();
    __threadfence();
    for (int tl = 0; tl < T; ++tl) {
        if (!last[tl])
            continue;
        for (int i = threadIdx.x; i < per_tile; i += blockDim.x) {
            int isum = 0;
            float fsum = 0.f;
            for (int sl = 0; sl < a.slices; ++sl) {
                const int pv = __ldcg(a.partials + ((size_t)sl * a.tiles + r_begin + tl) * (size_t)per_tile + i);
                if (GROUPED)
                    fsum += __int_as_float(pv);
                else
                    isum += pv;
            }
            finish(r_begin + tl, i >> 4, i & 15, GROUPED ? __float_as_int(fsum) : isum);
        }
    }
}

// ------------------------------------------------------------------------------------------- host side
template <int Q, int MT, int MP, bool GROUPED, int UW = 128>
static cudaError_t stream_launch_variant(const abq_gemm_state *st, const StreamArgs &args, cudaStream_t stream)
{
    auto kern = stream_kernel<Q, MT, MP, GROUPED, UW>;
    static thread_local SmemOptIn opted;
    cudaError_t e = opted.ensure(kern, st->shared_mem_size);
    if (e != cudaSuccess)
        return e;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(st->grid[0], 1, 1);
    cfg.blockDim = dim3(args.nw * 32);
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
    return cudaLaunchKernelEx(&cfg, kern, args);
}

template <int Q, int UW>
static cudaError_t stream_launch_grouped(const abq_gemm_state *st, const StreamArgs &args, int MT, int MP, cudaStream_t stream)
{
    if (MT == 4)
        return stream_launch_variant<Q, 4, 8, true, UW>(st, args, stream);
    if (MT == 2)
        return stream_launch_variant<Q, 2, 8, true, UW>(st, args, stream);
    switch (MP) {
    case 1: return stream_launch_variant<Q, 1, 1, true, UW>(st, args, stream);
    case 2: return stream_launch_variant<Q, 1, 2, true, UW>(st, args, stream);
    case 4: return stream_launch_variant<Q, 1, 4, true, UW>(st, args, stream);
    default: return stream_launch_variant<Q, 1, 8, true, UW>(st, args, stream);
    }
}

template <int Q>
static cudaError_t stream_launch_q(const abq_gemm_state *st, const StreamArgs &args, int MT, int MP, bool grouped, cudaStream_t stream)
{
    if (!grouped) {
        if (MT == 4)
            return stream_launch_variant<Q, 4, 8, false>(st, args, stream);
        if (MT == 2)
            return stream_launch_variant<Q, 2, 8, false>(st, args, stream);
        switch (MP) { // without group parameters the column blocks only make the activation records smaller
        case 1: return stream_launch_variant<Q, 1, 1, false>(st, args, stream);
        case 2: return stream_launch_variant<Q, 1, 2, false>(st, args, stream);
        case 4: return stream_launch_variant<Q, 1, 4, false>(st, args, stream);
        default: return stream_launch_variant<Q, 1, 8, false>(st, args, stream);
        }
    }
    return args.uw == 64 ? stream_launch_grouped<Q, 64>(st, args, MT, MP, stream) : stream_launch_grouped<Q, 128>(st, args, MT, MP, stream);
}

template <int Q>
static cudaError_t stream_prepare_q(const uint32_t *planes, const __half *w_scale, const uint8_t *w_zero, uint8_t *out, int N, int K, int w_signed,
                                    int grouped, int uw, int units_per_scale, int scale_groups, cudaStream_t stream)
{
    const long long threads = (long long)((N + 15) / 16) * (K / uw) * 32;
    const unsigned blocks = (unsigned)((threads + 255) / 256);
    if (uw == 64)
        prepare_stream_kernel<Q, 64><<<blocks, 256, 0, stream>>>(planes, w_scale, w_zero, out, N, K, w_signed, grouped, units_per_scale, scale_groups);
    else
        prepare_stream_kernel<Q, 128><<<blocks, 256, 0, stream>>>(planes, w_scale, w_zero, out, N, K, w_signed, grouped, units_per_scale, scale_groups);
    return cudaGetLastError();
}

// one definition per weight width, in gemm_stream_w<Q>.cu
#define ABQ_STREAM_WIDTH(Q)                                                                                                                     \
    cudaError_t stream_launch_w##Q(const abq_gemm_state *st, const StreamArgs &args, int MT, int MP, bool grouped, cudaStream_t stream)        \
    {                                                                                                                                           \
        return stream_launch_q<Q>(st, args, MT, MP, grouped, stream);                                                                           \
    }                                                                                                                                           \
    cudaError_t stream_prepare_w##Q(const uint32_t *planes, const __half *w_scale, const uint8_t *w_zero, uint8_t *out, int N, int K,          \
                                    int w_signed, int grouped, int uw, int units_per_scale, int scale_groups, cudaStream_t stream)             \
    {                                                                                                                                           \
        return stream_prepare_q<Q>(planes, w_scale, w_zero, out, N, K, w_signed, grouped, uw, units_per_scale, scale_groups, stream);           \
    }
#define ABQ_STREAM_DECLARE(Q)                                                                                                                   \
    cudaError_t stream_launch_w##Q(const abq_gemm_state *st, const StreamArgs &args, int MT, int MP, bool grouped, cudaStream_t stream);       \
    cudaError_t stream_prepare_w##Q(const uint32_t *planes, const __half *w_scale, const uint8_t *w_zero, uint8_t *out, int N, int K,          \
                                    int w_signed, int grouped, int uw, int units_per_scale, int scale_groups, cudaStream_t stream);
ABQ_STREAM_DECLARE(2)
ABQ_STREAM_DECLARE(3)
ABQ_STREAM_DECLARE(4)
ABQ_STREAM_DECLARE(8)

} // namespace abq
