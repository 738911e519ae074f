// Two-SM variant of the grouped block-scaled FP8 expert GEMM: a cluster of two CTAs computes one 256 x 256 output tile per
// K-block with tcgen05.mma.cta_group::2. Each CTA holds 128 rows of A and 128 of the 256 rows of B in its own shared memory
// and the tensor cores of both SMs read both halves, so every byte brought into shared memory feeds twice as many FLOPs as
// in the one-SM kernel (mf_moe_gemm_sm100.cu) — the one-SM kernel keeps the tensor pipe only ~30 % busy because filling
// shared memory, not the MMA, paces it. Same math contract as the one-SM kernel; used for large row counts (prefill).
//
// Roles per CTA (320 threads): warp 0 = TMA producer (per-CTA tiled 2-D loads, plain — no multicast — completing on the
// LEADER CTA's "full" barrier), warp 1 of the leader = MMA issuer (one thread; tcgen05.commit with a two-CTA arrival mask
// releases the shared-memory stage and publishes the partial product in both CTAs), warps 2-9 = promotion + epilogue on the
// CTA's own 128 TMEM lanes (256 accumulator columns, two buffers, 128 columns per thread). The peer's epilogue threads
// release a TMEM buffer by arriving on the leader's barrier through distributed shared memory. All waits are bounded.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "mf_kernels.h"
#include "mf_sm100_ptx.cuh"

using namespace mf::sm100;

namespace {

constexpr int BM = 128;        // rows of A per CTA (256 per pair)
constexpr int BNH = 128;       // rows of B per CTA (256 per pair)
constexpr int BN = 256;        // tile width
constexpr int BK = 128;
constexpr int kStages = 6;
constexpr int kThreads = 320;
constexpr int kEpiThreads = 256;
constexpr int kAccBufs = 2;
constexpr int kTileBytes = BM * BK;
constexpr int kMaxGroups = 256;
constexpr uint32_t kTmemCols = 512;

struct SharedStorage2 {
    alignas(1024) unsigned char a[kStages][kTileBytes];
    alignas(1024) unsigned char b[kStages][kTileBytes];
    uint64_t full[kStages];
    uint64_t empty[kStages];
    uint64_t tmemFull[kAccBufs];
    uint64_t tmemEmpty[kAccBufs];
    uint32_t tmemBase;
    int abortFlag;
    int tilePrefix[kMaxGroups + 1];
};

struct GemmParams2 {
    const float *aScale;
    const float *bScale;
    __nv_bfloat16 *out;
    const int *groupOffset;
    const int *groupCount;
    int *status;
    int G, N, K, mode, outStride;
};

__device__ __forceinline__ float Silu2(float x) { return x / (1.f + __expf(-x)); }

__device__ __forceinline__ uint32_t ClusterRank()
{
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t MapToCta(uint32_t smemAddr, uint32_t rank)
{
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smemAddr), "r"(rank));
    return r;
}
__device__ __forceinline__ void ClusterSync()
{
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void RemoteArrive(uint32_t clusterAddr)
{
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(clusterAddr) : "memory");
}
// Tiled 2-D load into this CTA's shared memory whose completion bytes are counted on a barrier that may live in the pair's
// other CTA (cta_group::2 form of the plain tiled load).
__device__ __forceinline__ void TmaLoad2DPair(void *smemDst, const CUtensorMap *m, uint32_t barClusterAddr, int c0, int c1)
{
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
                     SmemAddr(smemDst)),
                 "l"((uint64_t)m), "r"(barClusterAddr), "r"(c0), "r"(c1)
                 : "memory");
}
__device__ __forceinline__ void MmaF8Pair(uint32_t tmemD, uint64_t aDesc, uint64_t bDesc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n.reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n}\n" ::"r"(tmemD),
        "l"(aDesc), "l"(bDesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Arrives on the barrier at the same shared-memory offset in both CTAs of the pair once the MMAs issued so far are done.
__device__ __forceinline__ void MmaCommitPair(uint64_t *bar)
{
    const uint16_t mask = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(SmemAddr(bar)), "h"(mask)
                 : "memory");
}
__device__ __forceinline__ void TmemAllocPair(uint32_t *slot, uint32_t cols)
{
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(SmemAddr(slot)), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void TmemDeallocPair(uint32_t taddr, uint32_t cols)
{
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}

__global__ void __launch_bounds__(kThreads, 1)
mf_moe_grouped_gemm_2sm_kernel(const __grid_constant__ CUtensorMap tmapA, const __grid_constant__ CUtensorMap tmapB, const GemmParams2 p)
{
    extern __shared__ unsigned char smemRaw2[];
    SharedStorage2 &s = *reinterpret_cast<SharedStorage2 *>((reinterpret_cast<uintptr_t>(smemRaw2) + 1023) & ~(uintptr_t)1023);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t cta = ClusterRank();  // 0 = leader
    const int KB = p.K / BK, NT = p.N / BN;
    const int pairId = blockIdx.x >> 1, pairs = gridDim.x >> 1;

    if (threadIdx.x == 0) {
        for (int i = 0; i < kStages; i++) {
            MbarInit(&s.full[i], 1);
            MbarInit(&s.empty[i], 1);
        }
        for (int i = 0; i < kAccBufs; i++) {
            MbarInit(&s.tmemFull[i], 1);
            MbarInit(&s.tmemEmpty[i], 2 * kEpiThreads / 32);  // one arrival per epilogue warp of both CTAs, on the leader's copy
        }
        s.abortFlag = 0;
        int acc = 0;
        for (int g = 0; g < p.G; g++) {
            s.tilePrefix[g] = acc;
            acc += ((p.groupCount[g] + 2 * BM - 1) / (2 * BM)) * NT;
        }
        s.tilePrefix[p.G] = acc;
        MbarInitFence();
        TmaPrefetchDesc(&tmapA);
        TmaPrefetchDesc(&tmapB);
    }
    if (warp == 0) {
        TmemAllocPair(&s.tmemBase, kTmemCols);
    }
    TcFenceBefore();
    __syncthreads();
    ClusterSync();  // the peer's barriers exist before anybody signals them
    TcFenceAfter();
    const uint32_t tmemBase = s.tmemBase;
    const int totalTiles = s.tilePrefix[p.G];
    volatile int *abortFlag = &s.abortFlag;

    auto decode = [&](int tile, int &g, int &mt, int &nt) {
        int lo = 0, hi = p.G;
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (s.tilePrefix[mid] <= tile) {
                lo = mid;
            } else {
                hi = mid;
            }
        }
        g = lo;
        const int local = tile - s.tilePrefix[g];
        mt = local / NT;
        nt = local % NT;
    };

    if (warp == 0) {
        if (lane == 0) {
            const uint32_t leaderFull0 = MapToCta(SmemAddr(&s.full[0]), 0);
            uint32_t it = 0;
            for (int tile = pairId; tile < totalTiles && *abortFlag == 0; tile += pairs) {
                int g, mt, nt;
                decode(tile, g, mt, nt);
                const int rowA = p.groupOffset[g] + mt * 2 * BM + (int)cta * BM;
                const int rowB = g * p.N + nt * BN + (int)cta * BNH;
                for (int kb = 0; kb < KB; kb++, it++) {
                    const uint32_t st = it % kStages, ph = (it / kStages) & 1;
                    if (!MbarWaitBounded(&s.empty[st], ph ^ 1, abortFlag)) {
                        break;
                    }
                    if (p.mode & MF_GEMM_DEBUG_NO_LOADS) {
                        if (cta == 0) {
                            MbarArrive(&s.full[st]);
                        }
                        continue;
                    }
                    if (cta == 0) {
                        MbarExpectTx(&s.full[st], 4 * kTileBytes);  // A and B halves of both CTAs
                    }
                    const uint32_t bar = leaderFull0 + st * (uint32_t)sizeof(uint64_t);
                    TmaLoad2DPair(s.a[st], &tmapA, bar, kb * BK, rowA);
                    TmaLoad2DPair(s.b[st], &tmapB, bar, kb * BK, rowB);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && cta == 0) {
            constexpr uint32_t idesc = InstrDescF8(2 * BM, BN);
            uint32_t it = 0;
            for (int tile = pairId; tile < totalTiles && *abortFlag == 0; tile += pairs) {
                for (int kb = 0; kb < KB; kb++, it++) {
                    const uint32_t st = it % kStages, ph = (it / kStages) & 1;
                    const uint32_t buf = it % kAccBufs, bph = (it / kAccBufs) & 1;
                    if (!MbarWaitBounded(&s.tmemEmpty[buf], bph ^ 1, abortFlag) || !MbarWaitBounded(&s.full[st], ph, abortFlag)) {
                        break;
                    }
                    TcFenceAfter();
                    const uint64_t aDesc = SmemDescSw128(SmemAddr(s.a[st]));
                    const uint64_t bDesc = SmemDescSw128(SmemAddr(s.b[st]));
                    const uint32_t d = tmemBase + buf * BN;
#pragma unroll
                    for (int k = 0; k < BK / 32; k++) {
                        MmaF8Pair(d, aDesc + (uint64_t)(k * 2), bDesc + (uint64_t)(k * 2), idesc, k > 0 ? 1u : 0u);
                    }
                    MmaCommitPair(&s.empty[st]);
                    MmaCommitPair(&s.tmemFull[buf]);
                }
            }
        }
    } else {
        const int quad = warp & 3;
        const int half = (warp - 2) >> 2;  // 0: tile columns [0,128), 1: [128,256) — one 128-wide scale block each
        const int rowInTile = quad * 32 + lane;
        constexpr int HC = BN / 2;
        const uint32_t leaderEmpty0 = MapToCta(SmemAddr(&s.tmemEmpty[0]), 0);
        uint32_t it = 0;
        for (int tile = pairId; tile < totalTiles && *abortFlag == 0; tile += pairs) {
            int g, mt, nt;
            decode(tile, g, mt, nt);
            const int rowLocal = mt * 2 * BM + (int)cta * BM + rowInTile;
            const int row = p.groupOffset[g] + rowLocal;
            const bool valid = rowLocal < p.groupCount[g];
            const float *sa = p.aScale + (size_t)row * KB;
            const float *sb = p.bScale + ((size_t)g * (p.N / 128) + nt * 2 + half) * KB;
            float acc[HC];
#pragma unroll
            for (int i = 0; i < HC; i++) {
                acc[i] = 0.f;
            }
            float scaleNext = valid ? sa[0] * sb[0] : 0.f;
            bool ok = true;
            for (int kb = 0; kb < KB; kb++, it++) {
                const uint32_t buf = it % kAccBufs, bph = (it / kAccBufs) & 1;
                const float scale = scaleNext;
                if (kb + 1 < KB) {
                    scaleNext = valid ? sa[kb + 1] * sb[kb + 1] : 0.f;
                }
                if (!MbarWaitBounded(&s.tmemFull[buf], bph, abortFlag)) {
                    ok = false;
                    break;
                }
                TcFenceAfter();
                if (p.mode & MF_GEMM_DEBUG_NO_PROMOTION) {
                    TcFenceBefore();
                    __syncwarp();
                    if (lane == 0) {
                        RemoteArrive(leaderEmpty0 + buf * (uint32_t)sizeof(uint64_t));
                    }
                    continue;
                }
                const uint32_t taddr = tmemBase + ((uint32_t)(quad * 32) << 16) + buf * BN + half * HC;
#pragma unroll
                for (int c = 0; c < HC / 32; c++) {
                    float v[32];
                    TmemLd32Issue(taddr + c * 32, v);
                    TmemLdWait();
                    if (c == HC / 32 - 1) {
                        TcFenceBefore();
                        __syncwarp();
                        if (lane == 0) {
                            RemoteArrive(leaderEmpty0 + buf * (uint32_t)sizeof(uint64_t));  // the warp's part of the buffer is in registers
                        }
                    }
#pragma unroll
                    for (int i = 0; i < 32; i++) {
                        acc[c * 32 + i] = fmaf(v[i], scale, acc[c * 32 + i]);
                    }
                }
            }
            if (!ok) {
                break;
            }
            if (valid) {
                if ((p.mode & 15) == MF_GEMM_EPI_SWIGLU) {
                    // Each 64-column chunk holds 32 gate projections followed by the 32 matching up projections.
                    __nv_bfloat16 *o = p.out + (size_t)row * p.outStride + nt * (BN / 2) + half * (HC / 2);
#pragma unroll
                    for (int ch = 0; ch < HC / 64; ch++) {
#pragma unroll
                        for (int j = 0; j < 32; j += 8) {
                            uint4 pk;
                            __nv_bfloat162 *h = reinterpret_cast<__nv_bfloat162 *>(&pk);
#pragma unroll
                            for (int q = 0; q < 4; q++) {
                                const int gi = ch * 64 + j + 2 * q;
                                h[q] = __floats2bfloat162_rn(Silu2(acc[gi]) * acc[gi + 32], Silu2(acc[gi + 1]) * acc[gi + 33]);
                            }
                            *reinterpret_cast<uint4 *>(o + ch * 32 + j) = pk;
                        }
                    }
                } else {
                    __nv_bfloat16 *o = p.out + (size_t)row * p.outStride + nt * BN + half * HC;
#pragma unroll
                    for (int j = 0; j < HC; j += 8) {
                        uint4 pk;
                        __nv_bfloat162 *h = reinterpret_cast<__nv_bfloat162 *>(&pk);
#pragma unroll
                        for (int q = 0; q < 4; q++) {
                            h[q] = __floats2bfloat162_rn(acc[j + 2 * q], acc[j + 2 * q + 1]);
                        }
                        *reinterpret_cast<uint4 *>(o + j) = pk;
                    }
                }
            }
        }
    }
    TcFenceBefore();
    __syncthreads();
    if (s.abortFlag != 0 && threadIdx.x == 0 && p.status != nullptr) {
        atomicCAS(p.status, 0, 3);
    }
    ClusterSync();  // nobody leaves while the peer may still read its shared memory or signal its barriers
    if (warp == 0) {
        TcFenceAfter();
        TmemDeallocPair(tmemBase, kTmemCols);
    }
}

}  // namespace

// Launches the two-SM kernel. Same arguments as mf_k_moe_grouped_gemm; N must be a multiple of 256.
int mf_moe_grouped_gemm_2sm_launch(const CUtensorMap &mapA, const CUtensorMap &mapB, const float *aScale, const float *bScale, void *out,
                                   const int *groupOffset, const int *groupCount, int G, int N, int K, int mode, int *status, int ctas,
                                   cudaStream_t stream)
{
    GemmParams2 p;
    p.aScale = aScale;
    p.bScale = bScale;
    p.out = (__nv_bfloat16 *)out;
    p.groupOffset = groupOffset;
    p.groupCount = groupCount;
    p.status = status;
    p.G = G;
    p.N = N;
    p.K = K;
    p.mode = mode;
    p.outStride = (mode & 15) == MF_GEMM_EPI_SWIGLU ? N / 2 : N;
    static bool attrSet = false;
    const size_t smem = sizeof(SharedStorage2) + 1024;
    if (!attrSet) {
        if (cudaFuncSetAttribute(mf_moe_grouped_gemm_2sm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
            (void)cudaGetLastError();
            return MF_K_LAUNCH_FAILED;
        }
        attrSet = true;
    }
    int sms = mf_k_sm_count();
    if (sms < 2) {
        return MF_K_LAUNCH_FAILED;
    }
    int grid = (ctas > 1 && ctas < sms ? ctas : sms) & ~1;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((unsigned)grid, 1, 1);
    cfg.blockDim = dim3(kThreads, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, mf_moe_grouped_gemm_2sm_kernel, mapA, mapB, p);
    if (e != cudaSuccess) {
        (void)cudaGetLastError();
        return MF_K_LAUNCH_FAILED;
    }
    return MF_K_OK;
}
