// Device-side building blocks of the copy kernels: cache-hinted vector loads/stores and a CTA-cooperative span copy
// that handles any pair of byte alignments. Sources may be local HBM, a peer GPU's HBM mapped over NVLink, or pinned
// host memory; all are plain generic addresses in the global virtual address space.
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

namespace mf {
namespace dev {

// Streaming 16-byte load: read-only path, no L1 allocation (every byte is touched once).
__device__ __forceinline__ uint4 LdStream16(const void *p)
{
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ void StStream16(void *p, const uint4 &v)
{
    asm volatile("st.global.L1::no_allocate.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

template <typename T>
__device__ __forceinline__ T LdStream(const T *p)
{
    return *p;
}
template <>
__device__ __forceinline__ uint4 LdStream<uint4>(const uint4 *p)
{
    return LdStream16(p);
}
template <typename T>
__device__ __forceinline__ void StStream(T *p, const T &v)
{
    *p = v;
}
template <>
__device__ __forceinline__ void StStream<uint4>(uint4 *p, const uint4 &v)
{
    StStream16(p, v);
}

// Copies n elements of T with `nthreads` cooperating threads (this thread is `tid`), UNROLL independent loads in flight
// per thread before the first store.
template <typename T, int UNROLL>
__device__ __forceinline__ void CopyVec(T *__restrict__ dst, const T *__restrict__ src, size_t n, unsigned tid, unsigned nthreads)
{
    size_t i = tid;
    const size_t step = (size_t)nthreads * UNROLL;
    for (; i + (size_t)(UNROLL - 1) * nthreads < n; i += step) {
        T v[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; u++) {
            v[u] = LdStream<T>(src + i + (size_t)u * nthreads);
        }
#pragma unroll
        for (int u = 0; u < UNROLL; u++) {
            StStream<T>(dst + i + (size_t)u * nthreads, v[u]);
        }
    }
    for (; i < n; i += nthreads) {
        StStream<T>(dst + i, LdStream<T>(src + i));
    }
}

// Copies [src, src+n) to [dst, dst+n) with the threads (tid of nthreads). The destination is brought to a 16-byte
// boundary with byte stores; the body then uses the widest vector that the *relative* alignment of the two pointers
// allows (16 bytes when src and dst are congruent modulo 16).
template <int UNROLL>
__device__ __forceinline__ void CopySpan(unsigned char *dst, const unsigned char *src, size_t n, unsigned tid, unsigned nthreads)
{
    if (n == 0) {
        return;
    }
    size_t head = (16 - ((uintptr_t)dst & 15)) & 15;
    if (head > n) {
        head = n;
    }
    if (tid < head) {
        dst[tid] = src[tid];
    }
    dst += head;
    src += head;
    n -= head;
    const unsigned rel = (unsigned)((uintptr_t)src & 15);
    size_t body;
    if (rel == 0) {
        body = n & ~(size_t)15;
        CopyVec<uint4, UNROLL>((uint4 *)dst, (const uint4 *)src, body >> 4, tid, nthreads);
    } else if ((rel & 7) == 0) {
        body = n & ~(size_t)7;
        CopyVec<uint2, UNROLL>((uint2 *)dst, (const uint2 *)src, body >> 3, tid, nthreads);
    } else if ((rel & 3) == 0) {
        body = n & ~(size_t)3;
        CopyVec<uint32_t, UNROLL>((uint32_t *)dst, (const uint32_t *)src, body >> 2, tid, nthreads);
    } else if ((rel & 1) == 0) {
        body = n & ~(size_t)1;
        CopyVec<uint16_t, UNROLL>((uint16_t *)dst, (const uint16_t *)src, body >> 1, tid, nthreads);
    } else {
        body = n;
        CopyVec<unsigned char, UNROLL>(dst, src, body, tid, nthreads);
    }
    const size_t tail = n - body;
    if (tid < tail) {
        dst[body + tid] = src[body + tid];
    }
}

}  // namespace dev
}  // namespace mf
