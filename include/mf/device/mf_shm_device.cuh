/*
 * Device-side API of the symmetric heap: meta getters, peer addressing, put/get, signals with bounded waits and a
 * cross-rank barrier. Header-only; include it from your own .cu files and pass the pointer returned by
 * mf_shm_get_device_meta() to your kernel.
 *
 * Counterpart of the reference's AICore headers: meta getters (src/smem/include/device/smem_shm_aicore_base_meta.h:17-95),
 * scratchpad<->global copies (smem_shm_aicore_base_copy.h:17-113), in-kernel RDMA write/read/quiet
 * (smem_shm_aicore_base_rdma.h:132-376) and the flag helpers shown in its examples
 * (example/shm/AllReduce/shm_all_reduce.cpp:23-43). Inside one NVSwitch domain a peer's heap is ordinary global memory,
 * so put/get are plain 16-byte loads and stores and "quiet" is a system-scope fence. Unlike the reference's flag loop,
 * every wait here is bounded: on expiry it returns false and the caller records MF_DEV_ERR_TIMEOUT instead of hanging.
 */
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

struct alignas(128) MfDeviceMeta {
    uint32_t entityId;
    uint32_t rankId;
    uint32_t rankCount;
    uint32_t extraContextSize;
    uint64_t symmetricSize;
    uint64_t hbmBase;
    uint64_t dramBase;
    uint64_t dramWindowSize;
    uint64_t signalBase;
    uint64_t extraContextAddr;
    uint64_t multicastBase;
    uint64_t debugFlags; /* MF_DEBUG_* bits, set with mf_shm_set_debug_flags() or MF_CHECK_BOUNDS=1 */
    uint64_t reserved[6];
};

/* Debug aid for a platform without a device memory checker: with MF_DEBUG_CHECK_BOUNDS set in the heap's meta record, every
 * library kernel first checks that each argument which peers will address at the same heap offset (inputs they read, landing
 * zones they write) lies, with its full extent, inside THIS rank's window of the heap. A kernel whose arguments fail the check
 * touches no peer memory at all: it records MF_DEV_ERR_BOUNDS in its status word and returns. The check costs one branch per
 * kernel, so it may stay on in production runs that hunt a stray pointer. */
#define MF_DEBUG_CHECK_BOUNDS 1ull

/* Signal area of one rank (2 MiB): flags[channel][slot][rank] as 64-bit epochs, then scratch for library kernels. */
#define MF_SIGNAL_BYTES (2u * 1024u * 1024u)
#define MF_SIGNAL_CHANNELS 16u
#define MF_SIGNAL_SLOTS 64u
#define MF_SIGNAL_MAX_RANKS 64u
#define MF_SIGNAL_SCRATCH_OFFSET (512u * 1024u)

enum { MF_DEV_OK = 0, MF_DEV_ERR_TIMEOUT = 1, MF_DEV_ERR_BOUNDS = 2 };

__device__ __forceinline__ uint32_t mf_shm_get_global_rank(const MfDeviceMeta *m) { return m->rankId; }
__device__ __forceinline__ uint32_t mf_shm_get_global_rank_size(const MfDeviceMeta *m) { return m->rankCount; }
__device__ __forceinline__ uint64_t mf_shm_get_symmetric_size(const MfDeviceMeta *m) { return m->symmetricSize; }
__device__ __forceinline__ const void *mf_shm_get_extra_context_addr(const MfDeviceMeta *m) { return (const void *)m->extraContextAddr; }
__device__ __forceinline__ uint32_t mf_shm_get_extra_context_size(const MfDeviceMeta *m) { return m->extraContextSize; }

/* Address of heap offset `off` on `rank`. */
__device__ __forceinline__ void *mf_shm_ptr(const MfDeviceMeta *m, uint32_t rank, uint64_t off)
{
    return (void *)(m->hbmBase + (uint64_t)rank * m->symmetricSize + off);
}
/* The same heap offset as local pointer `p`, on `rank`. */
template <typename T>
__device__ __forceinline__ T *mf_shm_peer(const MfDeviceMeta *m, T *p, uint32_t rank)
{
    return (T *)((uint64_t)p + ((int64_t)rank - (int64_t)m->rankId) * (int64_t)m->symmetricSize);
}
/* Debug aid: true if [p, p+n) lies inside the heap of some rank. */
__device__ __forceinline__ bool mf_shm_in_heap(const MfDeviceMeta *m, const void *p, uint64_t n)
{
    uint64_t a = (uint64_t)p;
    return a >= m->hbmBase && a + n <= m->hbmBase + (uint64_t)m->rankCount * m->symmetricSize;
}

/* True if [p, p+n) lies inside the heap window of the calling rank (what peers address by offset must). */
__device__ __forceinline__ bool mf_shm_in_own_window(const MfDeviceMeta *m, const void *p, uint64_t n)
{
    const uint64_t a = (uint64_t)p, lo = m->hbmBase + (uint64_t)m->rankId * m->symmetricSize;
    return a >= lo && n <= m->symmetricSize && a + n <= lo + m->symmetricSize;
}
__device__ __forceinline__ bool mf_check_bounds_enabled(const MfDeviceMeta *m) { return (m->debugFlags & MF_DEBUG_CHECK_BOUNDS) != 0; }

__device__ __forceinline__ uint64_t *mf_signal_ptr(const MfDeviceMeta *m, uint32_t onRank, uint32_t channel, uint32_t slot, uint32_t fromRank)
{
    uint64_t base = m->signalBase + (uint64_t)onRank * MF_SIGNAL_BYTES;
    return (uint64_t *)base + ((uint64_t)channel * MF_SIGNAL_SLOTS + slot) * MF_SIGNAL_MAX_RANKS + fromRank;
}
__device__ __forceinline__ void *mf_signal_scratch(const MfDeviceMeta *m, uint32_t onRank)
{
    return (void *)(m->signalBase + (uint64_t)onRank * MF_SIGNAL_BYTES + MF_SIGNAL_SCRATCH_OFFSET);
}

__device__ __forceinline__ void mf_st_release_sys(uint64_t *p, uint64_t v)
{
    asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ uint64_t mf_ld_acquire_sys(const uint64_t *p)
{
    uint64_t v;
    asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint64_t mf_ld_relaxed_sys(const uint64_t *p)
{
    uint64_t v;
    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void mf_red_add_release_sys(uint64_t *p, uint64_t v)
{
    asm volatile("red.release.sys.global.add.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
/* Orders all earlier puts of the calling thread before its later signals (the reference's "quiet"). */
__device__ __forceinline__ void mf_quiet() { asm volatile("fence.acq_rel.sys;" ::: "memory"); }
__device__ __forceinline__ uint64_t mf_globaltimer_ns()
{
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

/* Signal: everything the calling thread wrote before is visible to whoever observes the value. */
__device__ __forceinline__ void mf_signal_set(uint64_t *remoteFlag, uint64_t value) { mf_st_release_sys(remoteFlag, value); }

/* Spins until *flag >= value or timeoutNs elapsed. Returns false on expiry (the caller records the error and leaves). */
__device__ __forceinline__ bool mf_wait_until_ge(const uint64_t *flag, uint64_t value, uint64_t timeoutNs)
{
    if (mf_ld_acquire_sys(flag) >= value) {
        return true;
    }
    const uint64_t t0 = mf_globaltimer_ns();
    uint32_t spins = 0;
    while (true) {
        if (mf_ld_acquire_sys(flag) >= value) {
            return true;
        }
        if ((++spins & 63u) == 0 && mf_globaltimer_ns() - t0 > timeoutNs) {
            return false;
        }
        __nanosleep(20);
    }
}

/* 16-byte streaming accessors for heap data.
 * mf_ld16 uses the non-coherent read-only path: legal only for data that nobody writes while the calling kernel runs
 * (inputs produced by earlier kernels of the stream). Data that another GPU, or another CTA, writes during the kernel and
 * that becomes visible through a signal or barrier inside the kernel must be read with mf_ld16_coherent. */
__device__ __forceinline__ uint4 mf_ld16(const void *p)
{
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
/* Coherent variant for data another GPU may have written during this kernel (after an acquire on a flag). */
__device__ __forceinline__ uint4 mf_ld16_coherent(const void *p)
{
    uint4 v;
    asm volatile("ld.relaxed.sys.global.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void mf_st16(void *p, const uint4 &v)
{
    asm volatile("st.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

/* CTA-cooperative put/get of n bytes; both addresses 16-byte aligned and n a multiple of 16. Call from all threads. */
__device__ __forceinline__ void mf_put16(void *remoteDst, const void *localSrc, uint64_t n)
{
    const uint64_t vecs = n >> 4;
    for (uint64_t i = threadIdx.x; i < vecs; i += blockDim.x) {
        mf_st16((char *)remoteDst + (i << 4), mf_ld16_coherent((const char *)localSrc + (i << 4)));
    }
}
__device__ __forceinline__ void mf_get16(void *localDst, const void *remoteSrc, uint64_t n) { mf_put16(localDst, remoteSrc, n); }

/*
 * Barrier across all ranks for ONE CTA per rank (the CTA with the same `slot` on every rank). Call from all threads of the
 * CTA with the same arguments on every rank; `epoch` must grow with every use of (channel, slot). Returns MF_DEV_OK or
 * MF_DEV_ERR_TIMEOUT | (peer << 8). Everything the CTA wrote before the call is visible to the peers' CTA after it.
 */
__device__ __forceinline__ int mf_barrier_cta(const MfDeviceMeta *m, uint32_t channel, uint32_t slot, uint64_t epoch, uint64_t timeoutNs)
{
    __shared__ int mf_bar_status;
    if (threadIdx.x == 0) {
        mf_bar_status = MF_DEV_OK;
    }
    __syncthreads();  // also: every thread's earlier writes happen-before thread t's release below
    const uint32_t n = m->rankCount, me = m->rankId;
    if (threadIdx.x < n) {
        const uint32_t peer = threadIdx.x;
        __threadfence_system();
        mf_signal_set(mf_signal_ptr(m, peer, channel, slot, me), epoch);
        if (!mf_wait_until_ge(mf_signal_ptr(m, me, channel, slot, peer), epoch, timeoutNs)) {
            atomicExch(&mf_bar_status, MF_DEV_ERR_TIMEOUT | (int)(peer << 8));
        }
    }
    __syncthreads();
    return mf_bar_status;
}

/* multimem (NVLS) accessors on the multicast alias of the heap: in-switch reduction and broadcast, bf16x2 lanes. */
__device__ __forceinline__ uint4 mf_multimem_ld_reduce_add_bf16x8(const void *mcAddr)
{
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(mcAddr)
                 : "memory");
    return v;
}
__device__ __forceinline__ void mf_multimem_st16(void *mcAddr, const uint4 &v)
{
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(mcAddr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
