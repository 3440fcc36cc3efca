// Device-side building blocks shared by the sm_100a kernels: mbarrier / TMA / cluster / PDL / MMA
// wrappers in inline PTX, the bounded-wait policy, and the bit-plane -> byte expansion.
#pragma once
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <stdint.h>

#include "../../include/abq_b200.h"

namespace abq {

// Device status word bits (written with atomicOr when a bounded wait expires).
enum : int {
    STATUS_TIMEOUT_TMA = 1,     // a TMA / bulk-copy completion barrier never flipped
    STATUS_TIMEOUT_PIPE = 2,    // a pipeline "stage free" barrier never flipped
    STATUS_TIMEOUT_MMA = 4,     // a tcgen05.commit barrier never flipped
    STATUS_TMEM_ALLOC = 8       // tcgen05.alloc did not return columns
};

// Upper bound for any spin in a kernel, in nanoseconds of %globaltimer.
constexpr unsigned long long kWaitLimitNs = 1000ull * 1000ull * 1000ull;

__device__ __forceinline__ uint32_t smem_u32(const void *p)
{
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ unsigned long long globaltimer_ns()
{
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// fp16 load for pointers that may be NULL in modes that never read them.  cuda_fp16's __ldg(const __half*)
// is a non-volatile inline-asm load, which the compiler is free to hoist above the branch guarding it (it
// did: a NULL scale pointer then faults in a mode that never uses it); a plain load is not speculated.
__device__ __forceinline__ __half ld_half(const __half *p)
{
    return __ushort_as_half(*reinterpret_cast<const unsigned short *>(p));
}

// ---------------------------------------------------------------- mbarrier
__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init()
{
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t *bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile("{\n"
                 ".reg .pred p;\n"
                 "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
                 "selp.u32 %0, 1, 0, p;\n"
                 "}\n"
                 : "=r"(ok)
                 : "r"(smem_u32(bar)), "r"(parity)
                 : "memory");
    return ok != 0;
}
// Wait for the phase with the given parity to complete.  Never spins for longer than kWaitLimitNs:
// on expiry the status bit is recorded (if a status word was given) and false is returned; the
// caller carries on to its exit path so that the kernel always terminates.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t *bar, uint32_t parity, int *status_word, int status_bit)
{
    if (mbar_try_wait(bar, parity))
        return true;
    const unsigned long long t0 = globaltimer_ns();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 64; ++i)
            if (mbar_try_wait(bar, parity))
                return true;
        if (globaltimer_ns() - t0 > kWaitLimitNs) {
            if (status_word)
                atomicOr(status_word, status_bit);
            return false;
        }
    }
}

// ---------------------------------------------------------------- async copies
__device__ __forceinline__ void fence_proxy_async()
{
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
// Contiguous global -> shared bulk copy (16-byte aligned addresses, size multiple of 16).
__device__ __forceinline__ void bulk_load(void *smem_dst, const void *gsrc, uint32_t bytes, uint64_t *bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(smem_dst)),
                 "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}
// Tiled TMA loads.  Coordinates are innermost first; the innermost one times the element size must be
// a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_2d(void *smem_dst, const void *tmap, int c0, int c1, uint64_t *bar)
{
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
                     smem_u32(smem_dst)),
                 "l"(tmap), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
                 : "memory");
}
__device__ __forceinline__ void tma_load_3d(void *smem_dst, const void *tmap, int c0, int c1, int c2, uint64_t *bar)
{
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];" ::"r"(
                     smem_u32(smem_dst)),
                 "l"(tmap), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2)
                 : "memory");
}
__device__ __forceinline__ void prefetch_tmap(const void *tmap)
{
    asm volatile("prefetch.tensormap [%0];" ::"l"(tmap) : "memory");
}

// ---------------------------------------------------------------- programmatic dependent launch
__device__ __forceinline__ void pdl_wait_prior_grid() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---------------------------------------------------------------- thread-block clusters
__device__ __forceinline__ uint32_t cluster_ctarank()
{
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t cluster_nctarank()
{
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_arrive_release() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait_acquire() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_sync_all()
{
    cluster_arrive_release();
    cluster_wait_acquire();
}
// Address of the same shared-memory location in another CTA of the cluster.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local_smem_addr, uint32_t cta_rank)
{
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_smem_addr), "r"(cta_rank));
    return r;
}
__device__ __forceinline__ uint4 ld_cluster_v4(uint32_t cluster_addr)
{
    uint4 v;
    asm volatile("ld.shared::cluster.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "r"(cluster_addr)
                 : "memory");
    return v;
}

// ---------------------------------------------------------------- legacy integer tensor-core MMA
// D(16x8, s32) += A(16x32, u8, row) * B(32x8, s8 or u8, col)
template <bool B_UNSIGNED>
__device__ __forceinline__ void mma_u8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                       uint32_t b1)
{
    if (B_UNSIGNED) {
        asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.u8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                     : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
                     : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    } else {
        asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                     : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
                     : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    }
}

// ---------------------------------------------------------------- bit-plane -> byte expansion
// Given the BITS plane words of 32 consecutive codes (plane b in p[b]), produce eight registers
// r[0..7]; byte y of r[s] is the unsigned code of the element stored at bit (8*y + s) of the words,
// i.e. element index j = 31 - 8*y - s of the 32-element run.  `flip_top` complements the top plane,
// which turns a two's complement code c into the offset code c + 2^(BITS-1).
template <int BITS>
__device__ __forceinline__ void planes_to_bytes(const uint32_t (&p)[BITS], bool flip_top, uint32_t (&r)[8])
{
#pragma unroll
    for (int s = 0; s < 8; ++s)
        r[s] = 0;
#pragma unroll
    for (int b = 0; b < BITS; ++b) {
        uint32_t w = p[b];
        if (b == BITS - 1 && flip_top)
            w = ~w;
#pragma unroll
        for (int s = 0; s < 8; ++s) {
            // move bit (8y + s) of w to bit (8y + b) of r[s]
            uint32_t t = (s >= b) ? (w >> (s - b)) : (w << (b - s));
            r[s] |= t & (0x01010101u << b);
        }
    }
}

// The inverse: eight registers of code bytes in the layout above -> the BITS plane words (bits above BITS ignored).
template <int BITS>
__device__ __forceinline__ void bytes_to_planes(const uint32_t (&r)[8], uint32_t (&p)[BITS])
{
#pragma unroll
    for (int b = 0; b < BITS; ++b) {
        uint32_t w = 0;
#pragma unroll
        for (int s = 0; s < 8; ++s) {
            // bit (8y + b) of r[s] goes to bit (8y + s) of the plane word
            const uint32_t t = (s >= b) ? (r[s] << (s - b)) : (r[s] >> (b - s));
            w |= t & (0x01010101u << s);
        }
        p[b] = w;
    }
}

// 8-bit lanes: (v ^ m) - m for every byte (sign extension of a BITS-wide two's complement field).
__device__ __forceinline__ uint32_t sign_extend_bytes(uint32_t v, int bits)
{
    const uint32_t m = 0x01010101u * (1u << (bits - 1));
    return __vsub4(v ^ m, m);
}

} // namespace abq
