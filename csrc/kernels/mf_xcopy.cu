// xcopy kernels: the data plane for every device-visible leg of a copy.
//
// mf_xcopy_kernel        one contiguous copy, any alignment. Contract of the reference's hybm_copy_kernel
//                        (src/hybm/csrc/copy_extend/hybm_copy_kernel.cpp:44-83): split the byte range over the grid in
//                        aligned shares and move each share load→store; bit-exact result.
// mf_batch_xcopy_kernel  N independent {src,dst,len} copies in one launch plus a completion word. Contract of
//                        hybm_batch_copy_kernel and its parameter-slot protocol (hybm_copy_kernel.cpp:85-124,
//                        src/hybm/csrc/data_operation/host/hybm_data_op_sdma.cpp:504-543). Differences by design:
//                        work is balanced by BYTES (fixed-size chunks found by binary search over a prefix table)
//                        rather than by descriptor index, small tables ride in the kernel parameters, and completion is
//                        one counter + one system-scope release store instead of a chain of blocks spinning on each other
//                        (no device-side wait exists in this kernel, so nothing can hang).
// Blackwell mapping: 16-byte streaming loads with L1 bypass, 8 loads in flight per thread before the first store,
// 512-thread CTAs at two per SM (128 KiB in flight per SM — enough to cover HBM3e and NVLink latency), persistent grid.
#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>

#include "mf_copy_device.cuh"
#include "mf_kernels.h"

namespace {

constexpr int kThreads = 512;
constexpr int kUnroll = 8;
constexpr size_t kPdlMaxBytes = 32 * 1024;

__global__ void __launch_bounds__(kThreads, 2)
mf_xcopy_kernel(unsigned char *__restrict__ dst, const unsigned char *__restrict__ src, size_t n, size_t tileBytes)
{
    // Programmatic dependent launch: when the host sets the stream-serialisation attribute (copies up to kPdlMaxBytes: beyond it the overlap measured no gain), the
    // next kernel of the stream may be scheduled while this one runs, and this kernel may have been scheduled while its
    // predecessor ran; the wait returns once the predecessor has completed and its writes are visible, so stream order
    // is kept and only the launch latency between back-to-back copies is hidden. Without the attribute both
    // instructions do nothing.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    // Tile 0 is stretched by `lead` bytes so that every later tile starts on a 16-byte boundary of dst.
    const size_t lead = (16 - ((uintptr_t)dst & 15)) & 15;
    const size_t body = n > lead ? n - lead : 0;
    const size_t ntiles = body == 0 ? 1 : (body + tileBytes - 1) / tileBytes;
    for (size_t t = blockIdx.x; t < ntiles; t += gridDim.x) {
        size_t begin = t == 0 ? 0 : lead + t * tileBytes;
        size_t end = lead + (t + 1) * tileBytes;
        if (end > n) {
            end = n;
        }
        mf::dev::CopySpan<kUnroll>(dst + begin, src + begin, end - begin, threadIdx.x, kThreads);
    }
}

// ---------------------------------------------------------------------------------------------- bulk-copy (TMA) variant
// For large copies whose two addresses are congruent modulo 16: each CTA streams tiles global → shared → global with the bulk
// asynchronous copy engine of the SM (cp.async.bulk, no tensor map, no multicast) through a ring of shared-memory stages. One
// thread issues loads, one thread issues stores; mbarriers hand tiles over. The SM's load/store units and register file stay out of the
// data path, so the copy runs at what the memory system and NVLink deliver. Waits are bounded like everywhere else.
// Default pipeline shapes, picked from a sweep of tile x stages x stores in flight x walk order x CTAs per SM on local HBM
// copies (a shallow pipeline interleaves DRAM reads and writes more regularly than a deep one: 6 stages with 3 stores in
// flight measured 3.11 TB/s at 1 GiB, the shapes below 3.30 TB/s, the copy engine 3.27 TB/s). Over NVLink every shape
// runs at the link's rate. Large copies: 32 KiB tiles, 4 stages, 2 stores in flight, each CTA on one contiguous run.
// Smaller ones: 16 KiB tiles, 4 stages, 1 store in flight, strided walk, two CTAs per SM so the last wave is short.
constexpr size_t kTmaLargeBytes = 256u << 20;

__device__ __forceinline__ uint32_t SmemU32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ bool MbarWaitParity(uint64_t *bar, uint32_t parity)
{
    for (uint32_t i = 0; i < (1u << 26); i++) {
        uint32_t ok;
        asm volatile(
            "{\n.reg .pred p;\n"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
            "selp.u32 %0, 1, 0, p;\n}\n"
            : "=r"(ok)
            : "r"(SmemU32(bar)), "r"(parity)
            : "memory");
        if (ok) {
            return true;
        }
    }
    return false;  // about a minute of polling: the caller stops issuing work
}

constexpr int kTmaMaxStages = 16;

// Shape of the bulk-copy pipeline: bytes per tile (a multiple of 16), tiles of shared memory per CTA, how many stores may
// still be reading shared memory before a tile is handed back to the loader, and whether a CTA walks the copy with a stride
// of the grid (0) or owns one contiguous run of tiles (1).
struct TmaShape {
    uint32_t tile;
    uint32_t stages;
    uint32_t inflight;
    uint32_t blocked;
};

__device__ __forceinline__ void BulkWaitRead(uint32_t inflight)
{
    switch (inflight) {
        case 1: asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory"); break;
        case 2: asm volatile("cp.async.bulk.wait_group.read 2;" ::: "memory"); break;
        case 3: asm volatile("cp.async.bulk.wait_group.read 3;" ::: "memory"); break;
        case 4: asm volatile("cp.async.bulk.wait_group.read 4;" ::: "memory"); break;
        case 6: asm volatile("cp.async.bulk.wait_group.read 6;" ::: "memory"); break;
        default: asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); break;
    }
}

__global__ void __launch_bounds__(128, 1)
mf_xcopy_tma_kernel(unsigned char *__restrict__ dst, const unsigned char *__restrict__ src, size_t n, TmaShape shape)
{
    extern __shared__ unsigned char tmaSmemRaw[];
    unsigned char *tiles = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(tmaSmemRaw) + 127) & ~(uintptr_t)127);
    __shared__ uint64_t full[kTmaMaxStages], empty[kTmaMaxStages];
    const uint32_t kTmaTile = shape.tile, kTmaStages = shape.stages, kTmaStoresInFlight = shape.inflight;
    // Unaligned head (up to the first 16-byte boundary of dst) and tail bytes go through ordinary loads/stores.
    const size_t head = n < 16 ? n : ((16 - ((uintptr_t)dst & 15)) & 15);
    const size_t body = (n - head) & ~(size_t)15;
    const size_t tail = n - head - body;
    if (blockIdx.x == 0 && threadIdx.x >= 64) {
        const unsigned t = threadIdx.x - 64;
        if (t < head) {
            dst[t] = src[t];
        }
        if (t < tail) {
            dst[head + body + t] = src[head + body + t];
        }
    }
    if (threadIdx.x == 0) {
        for (uint32_t i = 0; i < kTmaStages; i++) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(SmemU32(&full[i])));
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(SmemU32(&empty[i])));
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    const size_t ntiles = (body + kTmaTile - 1) / kTmaTile;
    const unsigned char *s0 = src + head;
    unsigned char *d0 = dst + head;
    // Strided walk: tile t belongs to CTA t % grid. Blocked walk: CTA b owns tiles [b*per, (b+1)*per).
    const size_t per = (ntiles + gridDim.x - 1) / gridDim.x;
    const size_t tBegin = shape.blocked ? (size_t)blockIdx.x * per : blockIdx.x;
    const size_t tEnd = shape.blocked ? (tBegin + per < ntiles ? tBegin + per : ntiles) : ntiles;
    const size_t tStep = shape.blocked ? 1 : gridDim.x;
    if (threadIdx.x == 0) {
        uint32_t it = 0;
        for (size_t t = tBegin; t < tEnd; t += tStep, it++) {
            const uint32_t st = it % kTmaStages, ph = (it / kTmaStages) & 1;
            if (!MbarWaitParity(&empty[st], ph ^ 1)) {
                break;
            }
            const size_t off = t * kTmaTile;
            const uint32_t bytes = (uint32_t)(body - off < kTmaTile ? body - off : kTmaTile);
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(SmemU32(&full[st])), "r"(bytes) : "memory");
            asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                             SmemU32(tiles + (size_t)st * kTmaTile)),
                         "l"(s0 + off), "r"(bytes), "r"(SmemU32(&full[st]))
                         : "memory");
        }
    } else if (threadIdx.x == 32) {
        uint32_t it = 0;
        for (size_t t = tBegin; t < tEnd; t += tStep, it++) {
            const uint32_t st = it % kTmaStages, ph = (it / kTmaStages) & 1;
            if (!MbarWaitParity(&full[st], ph)) {
                break;
            }
            const size_t off = t * kTmaTile;
            const uint32_t bytes = (uint32_t)(body - off < kTmaTile ? body - off : kTmaTile);
            asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(d0 + off), "r"(SmemU32(tiles + (size_t)st * kTmaTile)),
                         "r"(bytes)
                         : "memory");
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            // All but the newest kTmaStoresInFlight stores have finished reading shared memory: hand that tile back.
            BulkWaitRead(kTmaStoresInFlight);
            if (it >= kTmaStoresInFlight) {
                const uint32_t done = (it - kTmaStoresInFlight) % kTmaStages;
                asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(SmemU32(&empty[done])) : "memory");
            }
        }
        asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");  // every store has landed before the CTA retires
    }
}

struct BatchInline {
    uint32_t count;
    uint32_t totalChunks;
    uint32_t flagValue;
    uint32_t pad;
    uint32_t *doneCounter;
    volatile uint32_t *hostFlag;
    mf_copy_desc_t d[MF_BATCH_INLINE_MAX];
};
static_assert(sizeof(BatchInline) <= 4096 + 32, "inline batch must fit the classic kernel parameter space");

__device__ __forceinline__ void BatchBody(const mf_copy_desc_t *__restrict__ d, uint32_t count, uint32_t totalChunks,
                                          const uint32_t *__restrict__ chunkMap)
{
    for (uint32_t c = blockIdx.x; c < totalChunks; c += gridDim.x) {
        uint32_t lo = 0;
        if (chunkMap != nullptr) {
            lo = chunkMap[c];  // table in global memory: one load instead of a chain of dependent ones
        } else {
            // Last descriptor whose chunkStart <= c. The table sits in the constant bank (kernel parameters), all
            // threads search the same value: uniform, a few cycles per step.
            uint32_t hi = count;
            while (hi - lo > 1) {
                uint32_t mid = (lo + hi) >> 1;
                if (d[mid].chunkStart <= c) {
                    lo = mid;
                } else {
                    hi = mid;
                }
            }
        }
        const uint64_t off = (uint64_t)(c - d[lo].chunkStart) * MF_BATCH_CHUNK_BYTES;
        uint64_t len = d[lo].len - off;
        if (len > MF_BATCH_CHUNK_BYTES) {
            len = MF_BATCH_CHUNK_BYTES;
        }
        mf::dev::CopySpan<4>((unsigned char *)(d[lo].dst + off), (const unsigned char *)(d[lo].src + off), len, threadIdx.x, kThreads);
    }
}

__device__ __forceinline__ void BatchSignal(uint32_t *doneCounter, volatile uint32_t *hostFlag, uint32_t flagValue)
{
    if (doneCounter == nullptr) {
        return;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence_system();  // this CTA's copies are visible system-wide before it is counted
        unsigned prev = atomicAdd(doneCounter, 1u);
        if (prev == gridDim.x - 1) {
            *doneCounter = 0;  // self-reset for the next launch that uses this slot
            __threadfence_system();
            if (hostFlag != nullptr) {
                asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(hostFlag), "r"(flagValue) : "memory");
            }
        }
    }
}

__global__ void __launch_bounds__(kThreads, 2) mf_batch_xcopy_inline_kernel(const __grid_constant__ BatchInline p)
{
    BatchBody(p.d, p.count, p.totalChunks, nullptr);
    BatchSignal(p.doneCounter, p.hostFlag, p.flagValue);
}

// The chunk → descriptor map follows the descriptor table in the same device buffer.
__global__ void __launch_bounds__(kThreads, 2)
mf_batch_xcopy_table_kernel(const mf_copy_desc_t *__restrict__ d, uint32_t count, uint32_t totalChunks, uint32_t *doneCounter,
                            volatile uint32_t *hostFlag, uint32_t flagValue)
{
    BatchBody(d, count, totalChunks, reinterpret_cast<const uint32_t *>(d + count));
    BatchSignal(doneCounter, hostFlag, flagValue);
}

// ---------------------------------------------------------------------------------------------- test support

__host__ __device__ __forceinline__ uint64_t Mix64(uint64_t x)
{
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}

__host__ __device__ __forceinline__ unsigned char PatternByte(uint64_t seed, uint64_t index)
{
    uint64_t w = Mix64(seed ^ (index >> 3));
    return (unsigned char)(w >> ((index & 7) * 8));
}

__global__ void mf_fill_pattern_kernel(unsigned char *dst, size_t n, uint64_t seed)
{
    size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        dst[i] = PatternByte(seed, i);
    }
}

__global__ void mf_check_pattern_kernel(const unsigned char *buf, size_t n, uint64_t seed, unsigned long long *mismatch)
{
    size_t stride = (size_t)gridDim.x * blockDim.x;
    unsigned long long bad = 0;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        bad += buf[i] != PatternByte(seed, i);
    }
    if (bad) {
        atomicAdd(mismatch, bad);
    }
}

__global__ void mf_checksum_kernel(const unsigned char *buf, size_t n, unsigned long long *out)
{
    size_t stride = (size_t)gridDim.x * blockDim.x;
    size_t words = (n + 7) / 8;
    unsigned long long acc = 0;
    for (size_t w = (size_t)blockIdx.x * blockDim.x + threadIdx.x; w < words; w += stride) {
        uint64_t v = 0;
        size_t base = w * 8;
        for (int b = 0; b < 8 && base + b < n; b++) {
            v |= (uint64_t)buf[base + b] << (8 * b);
        }
        acc += Mix64(v ^ (uint64_t)w);
    }
    if (acc) {
        atomicAdd(out, acc);
    }
}

int SmCount()
{
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
        (void)cudaGetLastError();
        return 0;
    }
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) {
            (void)cudaGetLastError();
            return 0;
        }
        cached[dev] = n;
    }
    return cached[dev];
}

int LaunchResult()
{
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? MF_K_OK : MF_K_LAUNCH_FAILED;
}

}  // namespace

extern "C" int mf_k_sm_count(void) { return SmCount(); }

extern "C" int mf_k_memcpy_async(void *dst, const void *src, size_t n, mf_stream_t stream)
{
    return (int)cudaMemcpyAsync(dst, src, n, cudaMemcpyDefault, (cudaStream_t)stream);
}

static bool ShapeValid(const TmaShape &sh)
{
    return sh.tile >= 1024 && sh.tile % 16 == 0 && sh.stages >= 2 && sh.stages <= kTmaMaxStages && (uint64_t)sh.tile * sh.stages <= 220u * 1024 &&
           sh.inflight >= 1 && sh.inflight < sh.stages && (sh.inflight <= 4 || sh.inflight == 6) && sh.blocked <= 1;
}

static int LaunchTma(void *dst, const void *src, size_t n, const TmaShape &shape, int ctas, int sms, mf_stream_t stream)
{
    static size_t attrBytes = 0;
    const size_t smem = (size_t)shape.stages * shape.tile + 128;
    if (smem > attrBytes) {
        if (cudaFuncSetAttribute(mf_xcopy_tma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
            (void)cudaGetLastError();
            return MF_K_LAUNCH_FAILED;
        }
        attrBytes = smem;
    }
    size_t tiles = (n + shape.tile - 1) / shape.tile;
    const size_t perSm = smem <= 110u * 1024 ? 2 : 1;  // two CTAs fit an SM when their tiles take less than half its shared memory
    const size_t full = (size_t)sms * perSm;
    size_t grid = ctas > 0 ? (size_t)ctas : (tiles < full ? tiles : full);
    mf_xcopy_tma_kernel<<<(unsigned)grid, 128, smem, (cudaStream_t)stream>>>((unsigned char *)dst, (const unsigned char *)src, n, shape);
    return LaunchResult();
}

// The bulk-copy kernel with an explicit pipeline shape, for tuning sweeps. Same preconditions as the automatic path: both
// addresses congruent modulo 16. ctas 0 = one per SM.
extern "C" int mf_k_xcopy_shaped(void *dst, const void *src, size_t n, uint32_t tile, uint32_t stages, uint32_t inflight, uint32_t blocked,
                                 int ctas, mf_stream_t stream)
{
    const TmaShape shape{tile, stages, inflight, blocked};
    if (dst == nullptr || src == nullptr || n == 0 || ctas < 0 || !ShapeValid(shape) || ((((uintptr_t)dst) ^ ((uintptr_t)src)) & 15) != 0) {
        return MF_K_INVALID;
    }
    const int sms = SmCount();
    if (sms <= 0) {
        return MF_K_LAUNCH_FAILED;
    }
    return LaunchTma(dst, src, n, shape, ctas, sms, stream);
}

extern "C" int mf_k_xcopy(void *dst, const void *src, size_t n, int ctas, mf_stream_t stream)
{
    if (n == 0) {
        return MF_K_OK;
    }
    if (dst == nullptr || src == nullptr) {
        return MF_K_INVALID;
    }
    const int sms = SmCount();
    if (sms <= 0) {
        return MF_K_LAUNCH_FAILED;
    }
    static const bool useTma = []() {
        const char *e = getenv("MF_XCOPY_TMA");
        return !(e != nullptr && e[0] == '0');
    }();
    static const bool usePdl = []() {
        const char *e = getenv("MF_XCOPY_PDL");
        return !(e != nullptr && e[0] == '0');
    }();
    if (useTma && ctas >= 0 && n >= (4u << 20) && ((((uintptr_t)dst) ^ ((uintptr_t)src)) & 15) == 0) {
        // MF_XCOPY_SHAPE="tile,stages,inflight,blocked" overrides the pipeline shape (read once).
        static const TmaShape forced = []() {
            TmaShape sh{0, 0, 0, 0};
            const char *e = getenv("MF_XCOPY_SHAPE");
            unsigned a = 0, b = 0, c = 0, d = 0;
            if (e != nullptr && sscanf(e, "%u,%u,%u,%u", &a, &b, &c, &d) == 4) {
                TmaShape cand{a, b, c, d};
                if (ShapeValid(cand)) {
                    sh = cand;
                }
            }
            return sh;
        }();
        const TmaShape shape = forced.tile != 0 ? forced : (n >= kTmaLargeBytes ? TmaShape{32 * 1024, 4, 2, 1} : TmaShape{16 * 1024, 4, 1, 0});
        return LaunchTma(dst, src, n, shape, ctas, sms, stream);
    }
    if (ctas < 0) {
        ctas = -ctas == 1 ? 0 : -ctas;  // negative: force the load/store kernel (with |ctas| CTAs, -1 = automatic)
    }
    const size_t maxCtas = (size_t)sms * 2;
    // Tile = what one CTA moves per loop trip. Large copies use 64 KiB (8 × 16 B per thread); mid-size copies shrink the
    // tile so that every SM gets work; 8 KiB is the floor (one 16-byte vector per thread).
    size_t tile = 64 * 1024;
    while (tile > 8 * 1024 && n / tile < maxCtas) {
        tile >>= 1;
    }
    size_t ntiles = (n + tile - 1) / tile;
    size_t grid = ctas > 0 ? (size_t)ctas : (ntiles < maxCtas ? ntiles : maxCtas);
    // Back-to-back small copies are bound by the launch-to-launch gap, not by bytes: up to kPdlMaxBytes the kernel is
    // launched with programmatic stream serialisation (measured on two B200s over NVLink: 4.1 us -> 2.5-2.9 us per 4-16 KiB
    // copy, against 3.1-3.6 us for the copy engine; from 64 KiB on the overlap no longer pays).
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(kThreads);
    cfg.stream = (cudaStream_t)stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = (usePdl && n <= kPdlMaxBytes) ? 1 : 0;
    if (cudaLaunchKernelEx(&cfg, mf_xcopy_kernel, (unsigned char *)dst, (const unsigned char *)src, n, tile) != cudaSuccess) {
        (void)cudaGetLastError();
        return MF_K_LAUNCH_FAILED;
    }
    return MF_K_OK;
}

extern "C" int mf_k_batch_xcopy(const mf_copy_desc_t *descs, const mf_copy_desc_t *descsDev, uint32_t count, uint32_t totalChunks,
                                uint32_t *doneCounter, volatile uint32_t *hostFlag, uint32_t flagValue, int ctas, mf_stream_t stream)
{
    if (count == 0 || totalChunks == 0) {
        return MF_K_OK;
    }
    const int sms = SmCount();
    if (sms <= 0) {
        return MF_K_LAUNCH_FAILED;
    }
    unsigned maxCtas = (unsigned)sms * 2;
    unsigned grid = ctas > 0 ? (unsigned)ctas : (totalChunks < maxCtas ? totalChunks : maxCtas);
    if (count <= MF_BATCH_INLINE_MAX && descs != nullptr) {
        BatchInline p;
        p.count = count;
        p.totalChunks = totalChunks;
        p.flagValue = flagValue;
        p.pad = 0;
        p.doneCounter = doneCounter;
        p.hostFlag = hostFlag;
        for (uint32_t i = 0; i < count; i++) {
            p.d[i] = descs[i];
        }
        mf_batch_xcopy_inline_kernel<<<grid, kThreads, 0, (cudaStream_t)stream>>>(p);
        return LaunchResult();
    }
    if (descsDev == nullptr) {
        return MF_K_INVALID;
    }
    mf_batch_xcopy_table_kernel<<<grid, kThreads, 0, (cudaStream_t)stream>>>(descsDev, count, totalChunks, doneCounter, hostFlag, flagValue);
    return LaunchResult();
}

extern "C" int mf_k_fill_pattern(void *dst, size_t n, uint64_t seed, mf_stream_t stream)
{
    if (n == 0) {
        return MF_K_OK;
    }
    size_t blocks = (n + 255) / 256;
    if (blocks > 148 * 16) {
        blocks = 148 * 16;
    }
    mf_fill_pattern_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>((unsigned char *)dst, n, seed);
    return LaunchResult();
}

extern "C" int mf_k_check_pattern(const void *buf, size_t n, uint64_t seed, unsigned long long *mismatch, mf_stream_t stream)
{
    if (cudaMemsetAsync(mismatch, 0, sizeof(unsigned long long), (cudaStream_t)stream) != cudaSuccess) {
        return LaunchResult();
    }
    if (n == 0) {
        return MF_K_OK;
    }
    size_t blocks = (n + 255) / 256;
    if (blocks > 148 * 16) {
        blocks = 148 * 16;
    }
    mf_check_pattern_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>((const unsigned char *)buf, n, seed, mismatch);
    return LaunchResult();
}

extern "C" int mf_k_checksum(const void *buf, size_t n, unsigned long long *out, mf_stream_t stream)
{
    if (cudaMemsetAsync(out, 0, sizeof(unsigned long long), (cudaStream_t)stream) != cudaSuccess) {
        return LaunchResult();
    }
    if (n == 0) {
        return MF_K_OK;
    }
    size_t blocks = ((n + 7) / 8 + 255) / 256;
    if (blocks > 148 * 16) {
        blocks = 148 * 16;
    }
    mf_checksum_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>((const unsigned char *)buf, n, out);
    return LaunchResult();
}

extern "C" unsigned char mf_k_pattern_byte_host(uint64_t seed, uint64_t index) { return PatternByte(seed, index); }

extern "C" unsigned long long mf_k_checksum_host(const void *buf, size_t n)
{
    const unsigned char *p = (const unsigned char *)buf;
    size_t words = (n + 7) / 8;
    unsigned long long acc = 0;
    for (size_t w = 0; w < words; w++) {
        uint64_t v = 0;
        size_t base = w * 8;
        for (int b = 0; b < 8 && base + b < n; b++) {
            v |= (uint64_t)p[base + b] << (8 * b);
        }
        acc += Mix64(v ^ (uint64_t)w);
    }
    return acc;
}

// ---------------------------------------------------------------------------------------------- batch copy without any allocation
// See mf_xcopy_noalloc.h. The descriptor table, the chunk map and the completion counter of this variant live in the array
// below instead of in memory obtained from cudaMalloc. Every GPU that loads the library carries the array until exit.
#include "mf_xcopy_noalloc.h"

#include <cstdio>
#include <mutex>

namespace {

constexpr size_t kNoAllocHeader = 256;  // completion counter, padded so that the table stays 256-byte aligned
constexpr size_t kNoAllocBytes =
    kNoAllocHeader + (size_t)MF_NOALLOC_MAX_COPIES * sizeof(mf_copy_desc_t) + (size_t)MF_NOALLOC_MAX_CHUNKS * sizeof(uint32_t);

static __device__ __align__(256) unsigned char g_noAllocScratch[kNoAllocBytes];

// Host-side mirror of what is sent to the device. Static storage: the entry point must not touch the heap either.
mf_copy_desc_t g_noAllocDescs[MF_NOALLOC_MAX_COPIES];
uint32_t g_noAllocMap[MF_NOALLOC_MAX_CHUNKS];
std::mutex g_noAllocMu;
void *g_noAllocDevPtr[64] = {nullptr};  // device address of g_noAllocScratch, per device ordinal

}  // namespace

extern "C" int mf_batch_xcopy_noalloc(const uint64_t *srcs, const uint64_t *dsts, const uint64_t *sizes, uint32_t count, void *stream)
{
    if (count != 0 && (srcs == nullptr || dsts == nullptr || sizes == nullptr)) {
        fprintf(stderr, "mf_batch_xcopy_noalloc: null array\n");
        return MF_K_INVALID;
    }
    if (count > MF_NOALLOC_MAX_COPIES) {
        fprintf(stderr, "mf_batch_xcopy_noalloc: %u copies exceed the fixed limit of %d per call\n", count, (int)MF_NOALLOC_MAX_COPIES);
        return MF_K_TOO_LARGE;
    }
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
        (void)cudaGetLastError();
        return MF_K_LAUNCH_FAILED;
    }
    std::lock_guard<std::mutex> g(g_noAllocMu);
    // In host code the array's name is only a handle for the runtime, not an address a kernel can use: ask the runtime
    // for the device address once per device, with that device current.
    if (g_noAllocDevPtr[dev] == nullptr) {
        void *p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_noAllocScratch);
        if (e != cudaSuccess || p == nullptr) {
            fprintf(stderr, "mf_batch_xcopy_noalloc: cudaGetSymbolAddress failed: %s\n", cudaGetErrorString(e));
            (void)cudaGetLastError();
            return MF_K_LAUNCH_FAILED;
        }
        g_noAllocDevPtr[dev] = p;
    }
    if (count == 0) {
        return MF_K_OK;  // warm-up call: the module is loaded and the array's address is known from here on
    }
    cudaStreamCaptureStatus capture = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing((cudaStream_t)stream, &capture) != cudaSuccess) {
        (void)cudaGetLastError();
        return MF_K_LAUNCH_FAILED;
    }
    if (capture != cudaStreamCaptureStatusNone) {
        fprintf(stderr, "mf_batch_xcopy_noalloc: the stream is being captured; the staged copy table cannot be part of a graph\n");
        return MF_K_INVALID;
    }
    unsigned char *base = static_cast<unsigned char *>(g_noAllocDevPtr[dev]);
    uint64_t chunks = 0;
    for (uint32_t i = 0; i < count; i++) {
        if (sizes[i] == 0 || sizes[i] >= (1ull << 32) || srcs[i] == 0 || dsts[i] == 0) {
            fprintf(stderr, "mf_batch_xcopy_noalloc: copy %u has a null address or a size outside 1 .. 4 GiB-1\n", i);
            return MF_K_INVALID;
        }
        const uint64_t n = (sizes[i] + MF_BATCH_CHUNK_BYTES - 1) / MF_BATCH_CHUNK_BYTES;
        if (chunks + n > MF_NOALLOC_MAX_CHUNKS) {
            fprintf(stderr, "mf_batch_xcopy_noalloc: the batch needs more than %d chunks of %d bytes (about %d MiB in total)\n",
                    (int)MF_NOALLOC_MAX_CHUNKS, (int)MF_BATCH_CHUNK_BYTES, (int)((uint64_t)MF_NOALLOC_MAX_CHUNKS * MF_BATCH_CHUNK_BYTES >> 20));
            return MF_K_TOO_LARGE;
        }
        g_noAllocDescs[i] = mf_copy_desc_t{srcs[i], dsts[i], (uint32_t)sizes[i], (uint32_t)chunks};
        for (uint64_t c = 0; c < n; c++) {
            g_noAllocMap[chunks + c] = i;
        }
        chunks += n;
    }
    cudaStream_t s = (cudaStream_t)stream;
    const size_t descBytes = (size_t)count * sizeof(mf_copy_desc_t);
    // The array keeps whatever the previous call left in it: the counter has to start at zero, the table and the map are
    // overwritten for exactly the part this call uses.
    if (cudaMemsetAsync(base, 0, kNoAllocHeader, s) != cudaSuccess ||
        cudaMemcpyAsync(base + kNoAllocHeader, g_noAllocDescs, descBytes, cudaMemcpyHostToDevice, s) != cudaSuccess ||
        cudaMemcpyAsync(base + kNoAllocHeader + descBytes, g_noAllocMap, (size_t)chunks * sizeof(uint32_t), cudaMemcpyHostToDevice, s) != cudaSuccess) {
        fprintf(stderr, "mf_batch_xcopy_noalloc: staging the copy table failed: %s\n", cudaGetErrorString(cudaGetLastError()));
        return MF_K_LAUNCH_FAILED;
    }
    const int sms = SmCount();
    if (sms <= 0) {
        return MF_K_LAUNCH_FAILED;
    }
    const unsigned maxCtas = (unsigned)sms * 2;
    const unsigned grid = chunks < maxCtas ? (unsigned)chunks : maxCtas;
    mf_batch_xcopy_table_kernel<<<grid, kThreads, 0, s>>>(reinterpret_cast<const mf_copy_desc_t *>(base + kNoAllocHeader), count, (uint32_t)chunks,
                                                         reinterpret_cast<uint32_t *>(base), nullptr, 0);
    return LaunchResult();
}
