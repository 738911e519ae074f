// Thin inline-PTX wrappers for the Blackwell (sm_100a) features the GEMM kernels use: mbarriers, TMA tiled loads
// (cp.async.bulk.tensor, never with cluster multicast), tensor memory (TMEM) management, tcgen05.mma / commit / ld and
// the shared-memory and instruction descriptors they take. Every wait is bounded: the *_bounded helpers return false when
// the iteration limit is hit so that the caller can flag an error and unwind (free TMEM, leave) instead of hanging.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace mf {
namespace sm100 {

__device__ __forceinline__ uint32_t SmemAddr(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

// ---------------------------------------------------------------------------------------------- mbarrier
__device__ __forceinline__ void MbarInit(uint64_t *bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(SmemAddr(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void MbarInitFence() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void MbarExpectTx(uint64_t *bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(SmemAddr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void MbarArrive(uint64_t *bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(SmemAddr(bar)) : "memory");
}
__device__ __forceinline__ bool MbarTryWait(uint64_t *bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n.reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(ok)
        : "r"(SmemAddr(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ uint64_t GlobalTimerNs()
{
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// Waits for the phase with the given parity; gives up after about limitNs (counted on the SM's cycle counter at two cycles
// per nanosecond, so between limitNs and twice that when the clock is low) or when *abortFlag becomes non-zero. On expiry it
// raises *abortFlag so that the other roles of the CTA unwind too. The wait sits on the hand-shake path of every pipeline
// stage, so the common case stays cheap: the counter and the flag are looked at once per 256 polls, and the global
// nanosecond timer (slow to read) not at all.
__device__ __forceinline__ bool MbarWaitBounded(uint64_t *bar, uint32_t parity, volatile int *abortFlag, uint64_t limitNs = 2000000000ull)
{
    if (MbarTryWait(bar, parity)) {
        return true;
    }
    long long t0 = 0;
    for (uint32_t i = 1; i < (1u << 30); i++) {
        if (MbarTryWait(bar, parity)) {
            return true;
        }
        if ((i & 255u) == 0u) {
            if (*abortFlag != 0) {
                return false;
            }
            const long long now = clock64();
            if (t0 == 0) {
                t0 = now;
            } else if ((uint64_t)(now - t0) > 2 * limitNs) {
                break;
            }
        }
    }
    *abortFlag = 1;
    return false;
}

// One 32-byte store (a whole sector) to global memory; the address must be 32-byte aligned.
__device__ __forceinline__ void StGlobal32B(void *p, const uint32_t (&w)[8])
{
    asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(p), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]), "r"(w[4]), "r"(w[5]),
                 "r"(w[6]), "r"(w[7])
                 : "memory");
}

// ---------------------------------------------------------------------------------------------- TMA
__device__ __forceinline__ void TmaPrefetchDesc(const CUtensorMap *m)
{
    asm volatile("prefetch.tensormap [%0];" ::"l"((uint64_t)m) : "memory");
}
// 2-D tiled load global → shared (this CTA), completion counted in bytes on `bar`. c0 is the innermost coordinate: its
// byte offset must be a multiple of 16.
__device__ __forceinline__ void TmaLoad2D(void *smemDst, const CUtensorMap *m, uint64_t *bar, int c0, int c1)
{
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(SmemAddr(smemDst)),
                 "l"((uint64_t)m), "r"(SmemAddr(bar)), "r"(c0), "r"(c1)
                 : "memory");
}
// The same for a 4-D tensor map (c0 innermost).
__device__ __forceinline__ void TmaLoad4D(void *smemDst, const CUtensorMap *m, uint64_t *bar, int c0, int c1, int c2, int c3)
{
    asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];" ::"r"(
                     SmemAddr(smemDst)),
                 "l"((uint64_t)m), "r"(SmemAddr(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
                 : "memory");
}

// ---------------------------------------------------------------------------------------------- TMEM
// Allocates `cols` (power of two, >= 32) TMEM columns; the base address is written to *smemSlot. Whole warp must call.
__device__ __forceinline__ void TmemAlloc(uint32_t *smemSlot, uint32_t cols)
{
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(SmemAddr(smemSlot)), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void TmemDealloc(uint32_t taddr, uint32_t cols)
{
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void TcFenceBefore() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void TcFenceAfter() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// Issues a load of 32 consecutive fp32 columns of this thread's TMEM lane (warp w reads lanes 32*(w%4) .. +31) straight
// into v[0..31]; the values may only be used after TmemLdWait().
__device__ __forceinline__ void TmemLd32Issue(uint32_t taddr, float *v)
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=f"(v[0]), "=f"(v[1]), "=f"(v[2]), "=f"(v[3]), "=f"(v[4]), "=f"(v[5]), "=f"(v[6]), "=f"(v[7]), "=f"(v[8]), "=f"(v[9]), "=f"(v[10]),
          "=f"(v[11]), "=f"(v[12]), "=f"(v[13]), "=f"(v[14]), "=f"(v[15]), "=f"(v[16]), "=f"(v[17]), "=f"(v[18]), "=f"(v[19]), "=f"(v[20]),
          "=f"(v[21]), "=f"(v[22]), "=f"(v[23]), "=f"(v[24]), "=f"(v[25]), "=f"(v[26]), "=f"(v[27]), "=f"(v[28]), "=f"(v[29]), "=f"(v[30]),
          "=f"(v[31])
        : "r"(taddr)
        : "memory");
}
// Same for 16 consecutive columns.
__device__ __forceinline__ void TmemLd16Issue(uint32_t taddr, float *v)
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=f"(v[0]), "=f"(v[1]), "=f"(v[2]), "=f"(v[3]), "=f"(v[4]), "=f"(v[5]), "=f"(v[6]), "=f"(v[7]), "=f"(v[8]), "=f"(v[9]), "=f"(v[10]),
          "=f"(v[11]), "=f"(v[12]), "=f"(v[13]), "=f"(v[14]), "=f"(v[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void TmemLdWait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// 32 consecutive fp32 columns of this thread's TMEM lane, waited for.
__device__ __forceinline__ void TmemLd32(uint32_t taddr, float *v)
{
    uint32_t r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]),
          "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
          "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]),
          "=r"(r[31])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; i++) {
        v[i] = __uint_as_float(r[i]);
    }
}

// ---------------------------------------------------------------------------------------------- descriptors
// Shared-memory matrix descriptor for a K-major tile stored as rows of 128 bytes with the 128-byte swizzle (what a TMA
// load with CU_TENSOR_MAP_SWIZZLE_128B produces): 8-row groups are 1024 bytes apart. Fields: start address >> 4 in bits
// [0,14), leading byte offset >> 4 in [16,30) (unused for this layout), stride byte offset >> 4 in [32,46), descriptor
// version 1 in [46,48), layout type 2 (SWIZZLE_128B) in [61,64).
__device__ __forceinline__ uint64_t SmemDescSw128(uint32_t smemByteAddr)
{
    uint64_t d = 0;
    d |= (uint64_t)((smemByteAddr & 0x3FFFFu) >> 4);
    d |= (uint64_t)(1024u >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

// Instruction descriptor for kind::f8f6f4, E4M3 x E4M3 -> F32, both operands K-major: D format F32 = 1 at [4,6), A format at
// [7,10), B format at [10,13) (0 = E4M3), A/B major at bits 15/16 (0 = K), N >> 3 at [17,23), M >> 4 at [24,29).
__host__ __device__ constexpr uint32_t InstrDescF8(uint32_t m, uint32_t n) { return (1u << 4) | ((n >> 3) << 17) | ((m >> 4) << 24); }
// Same for kind::f16 with BF16 operands (A/B format 1).
__host__ __device__ constexpr uint32_t InstrDescBf16(uint32_t m, uint32_t n)
{
    return (1u << 4) | (1u << 7) | (1u << 10) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

// D[tmem] (+)= A[smem] * B[smem], issued by ONE thread. accumulate = 0 overwrites D.
__device__ __forceinline__ void MmaF8(uint32_t tmemD, uint64_t aDesc, uint64_t bDesc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n.reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n}\n" ::"r"(tmemD),
        "l"(aDesc), "l"(bDesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// ---------------------------------------------------------------------------------------------- block-scaled MMA (kind::mxf8f6f4)
// Scale factors are UE8M0 bytes (value = 2^(byte - 127)), one per operand row and 32 K-elements. The tensor core reads them
// from TMEM: row r of a 128-row operand tile sits in lane r % 32 (replicated in all four 32-lane quadrants), 32-bit column
// r / 32 of the scale-factor area, and byte j of that column belongs to the j-th 32-element K step of a 128-element K block
// (selected per instruction through the a_sf_id / b_sf_id fields of the descriptor).

// Shared-memory descriptor of one scale-factor atom for tcgen05.cp: 32 rows of 16 bytes, no swizzle, 8-row groups 128 bytes apart.
__device__ __forceinline__ uint64_t SmemDescSfAtom(uint32_t smemByteAddr)
{
    uint64_t d = 0;
    d |= (uint64_t)((smemByteAddr & 0x3FFFFu) >> 4);
    d |= (uint64_t)(128u >> 4) << 32;
    d |= (uint64_t)1 << 46;
    return d;
}
// Copies one 512-byte scale-factor atom (32 rows x 16 bytes) from shared memory into four TMEM columns starting at `taddr`,
// replicated into the four lane quadrants. Issued by ONE thread; ordered with the tcgen05.mma that the same thread issues next.
__device__ __forceinline__ void TmemCpSfAtom(uint32_t taddr, uint64_t smemDesc)
{
    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(smemDesc) : "memory");
}
// Generic-proxy writes to shared memory (ordinary stores) become visible to the async proxy (tcgen05.cp, TMA) after this fence.
__device__ __forceinline__ void FenceProxyAsyncShared() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
// Orders global-memory accesses of the generic proxy (an acquire load that saw another agent's stores) before TMA reads.
__device__ __forceinline__ void FenceProxyAsyncGlobal() { asm volatile("fence.proxy.async.global;" ::: "memory"); }

// Instruction descriptor for kind::mxf8f6f4.block_scale, E4M3 x E4M3 (A/B format 0 at [7,10) and [10,13)), both operands K-major,
// UE8M0 scale factors (bit 23), N >> 3 at [17,23), M >> 4 at [24,29), byte selectors of the scale-factor columns: B at [4,6), A at
// [29,31). The accumulator is always fp32.
__host__ __device__ constexpr uint32_t InstrDescMxF8(uint32_t m, uint32_t n, uint32_t sfId)
{
    return (sfId << 4) | (1u << 23) | ((n >> 3) << 17) | ((m >> 4) << 24) | (sfId << 29);
}
// D[tmem] (+)= (A * sfa) x (B * sfb)^T for one 32-element K step, issued by ONE thread. sfaTmem / sfbTmem: TMEM addresses of the
// scale-factor columns (the byte selector travels in the descriptor).
__device__ __forceinline__ void MmaMxF8(uint32_t tmemD, uint64_t aDesc, uint64_t bDesc, uint32_t idesc, uint32_t sfaTmem, uint32_t sfbTmem,
                                        uint32_t accumulate)
{
    asm volatile(
        "{\n.reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n}\n" ::"r"(tmemD),
        "l"(aDesc), "l"(bDesc), "r"(idesc), "r"(accumulate), "r"(sfaTmem), "r"(sfbTmem)
        : "memory");
}
// Makes `bar` complete once all tcgen05.mma issued so far by this thread have finished (implies fence::before_thread_sync).
__device__ __forceinline__ void MmaCommit(uint64_t *bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(SmemAddr(bar)) : "memory");
}

}  // namespace sm100
}  // namespace mf
