// Two-SM form of the block-scaled grouped FP8 expert GEMM (see mf_moe_gemm_mx_sm100.cu for the math contract and the operand
// formats): a cluster of two CTAs computes one 256 x 256 output tile with tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale.
// Each CTA brings 128 rows of A and 128 of the tile's 256 weight rows into its own shared memory and the tensor cores of both
// SMs read both halves, so a K block costs each SM 32 KiB of operand traffic instead of the 48 KiB of the one-SM 128 x 256 tile:
// one third less shared-memory fill per FLOP, and a ring of six stages instead of four in the same shared memory, i.e. more K
// blocks in flight to cover the latency of L2 and DRAM. The one-SM kernel keeps the tensor pipe about 60 % busy with L2, DRAM
// and the TMA unit all below 40 % of their peaks; the fill latency, not a throughput limit, paces it. Measured, the pair's longer
// hand-shakes (commit to both CTAs, byte counts and arrivals crossing to the leader) cost what the deeper ring gains: 0.89 ms
// against 0.83 ms for the one-SM kernel on the first FFN GEMM of the benchmark, equal on the second; the one-SM kernel stays
// the default.
//
// Roles per CTA (384 threads): warp 0 TMA producer (per-CTA tiled loads, no multicast, completing on the LEADER's "full"
// barrier), warp 2 scale-factor producer (this CTA's 128 A rows, all 256 weight columns; the atoms have a ring of their own —
// two groups of four K blocks, one hand-shake per group on the leader's "sfFull" — so that the operand ring turns on the TMA
// loads alone and no remote arrival sits in its revolution), warp 1 of the leader issues the scale-factor copies (alternating
// between two sets of TMEM columns) and the MMAs for the pair; tcgen05.commit with a two-CTA mask releases the stage (and, per
// group, the atoms) and publishes the accumulator in both CTAs; warps 4-11 run the epilogue on the CTA's own 128 TMEM lanes and
// release the accumulator by arriving on the leader's barrier (through distributed shared memory from the second CTA). Every
// wait is bounded.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

#include <cstdlib>

#include "mf_kernels.h"
#include "mf_sm100_ptx.cuh"

using namespace mf::sm100;

namespace {

constexpr int BM = 128;   // A rows per CTA (256 per pair)
constexpr int BNH = 128;  // weight rows per CTA (256 per pair)
constexpr int BN = 256;
constexpr int BK = 128;
constexpr int kStages = 6;
constexpr int kThreads = 384;
constexpr int kEpiWarps = 8;
constexpr int kMaxGroups = 256;
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kSfaCol = 256;  // [0, 256) accumulator, [256, 260) A scale factors, [260, 268) weight scale factors,
constexpr uint32_t kSfbCol = 260;  // [268, 280) a second set of both: K blocks alternate
constexpr uint32_t kSfSetCols = 12;
constexpr uint32_t kSfOne = 0x7f7f7f7fu;
constexpr int kSfGroup = 4;             // K blocks whose scale atoms are produced and released together
constexpr int kSfSlots = 2 * kSfGroup;  // two groups: one being consumed, one being filled
constexpr int kTileBytes = BM * BK;

struct SharedStorage2 {
    alignas(1024) unsigned char a[kStages][kTileBytes];
    alignas(1024) unsigned char b[kStages][kTileBytes];
    alignas(128) unsigned char sfa[kSfSlots][512];
    alignas(128) unsigned char sfb[kSfSlots][1024];
    uint64_t full[kStages];   // used in the leader: TMA bytes of both CTAs
    uint64_t empty[kStages];  // one copy per CTA, released together by the commit
    uint64_t sfFull[2];       // used in the leader: the scale-factor warps of both CTAs
    uint64_t sfEmpty[2];      // one copy per CTA, released together by the commit
    uint64_t tmemFull;        // one copy per CTA
    uint64_t tmemEmpty;       // used in the leader: epilogue warps of both CTAs
    uint32_t tmemBase;
    int abortFlag;
    int tilePrefix[kMaxGroups + 1];
};

struct Mx2Params {
    const uint32_t *aSf;
    const float *bScale;
    void *out;
    unsigned char *outSf;
    const int *groupOffset;
    const int *groupCount;
    int *status;
    int G, N, K, mode, rowsTotal;
    int wideStores;  // out is 32-byte aligned: the epilogue stores whole sectors
};

__device__ __forceinline__ float Silu(float x) { return x / (1.f + __expf(-x)); }

__device__ __forceinline__ uint32_t Ue8m0Ceil(float t)
{
    const uint32_t bits = __float_as_uint(t);
    uint32_t e = ((bits >> 23) & 0xffu) + ((bits & 0x7fffffu) != 0u ? 1u : 0u);
    return e < 1u ? 1u : (e > 253u ? 253u : e);
}

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
// Tiled 2-D load into THIS CTA's shared memory whose bytes are counted on a barrier that may live in the pair's other CTA.
__device__ __forceinline__ void TmaLoad2DPair(void *smemDst, const CUtensorMap *m, uint32_t barClusterAddr, int c0, int c1)
{
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
                     SmemAddr(smemDst)),
                 "l"((uint64_t)m), "r"(barClusterAddr), "r"(c0), "r"(c1)
                 : "memory");
}
__device__ __forceinline__ void MmaMxF8Pair(uint32_t tmemD, uint64_t aDesc, uint64_t bDesc, uint32_t idesc, uint32_t sfaTmem, uint32_t sfbTmem,
                                            uint32_t accumulate)
{
    asm volatile(
        "{\n.reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n}\n" ::"r"(tmemD),
        "l"(aDesc), "l"(bDesc), "r"(idesc), "r"(accumulate), "r"(sfaTmem), "r"(sfbTmem)
        : "memory");
}
// Copies a scale-factor atom from shared memory to TMEM in BOTH CTAs (each from its own shared memory, same offsets).
__device__ __forceinline__ void TmemCpSfAtomPair(uint32_t taddr, uint64_t smemDesc)
{
    asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(smemDesc) : "memory");
}
// Arrives on the barrier at the same shared-memory offset in both CTAs once the operations issued so far are done.
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
mf_moe_grouped_gemm_mx2_kernel(const __grid_constant__ CUtensorMap tmapA, const __grid_constant__ CUtensorMap tmapB, const Mx2Params p)
{
    extern __shared__ unsigned char smemRaw[];
    SharedStorage2 &s = *reinterpret_cast<SharedStorage2 *>((reinterpret_cast<uintptr_t>(smemRaw) + 1023) & ~(uintptr_t)1023);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t cta = ClusterRank();  // 0 = leader
    const int KB = p.K / BK, NT = p.N / BN;
    const int pairId = blockIdx.x >> 1, pairs = gridDim.x >> 1;

    for (int g = threadIdx.x; g < p.G; g += kThreads) {
        s.tilePrefix[g + 1] = ((p.groupCount[g] + 2 * BM - 1) / (2 * BM)) * NT;
    }
    if (threadIdx.x == 0) {
        for (int i = 0; i < kStages; i++) {
            MbarInit(&s.full[i], 1);  // the leader's TMA thread, with the byte count of both CTAs
            MbarInit(&s.empty[i], 1);
        }
        for (int i = 0; i < 2; i++) {
            MbarInit(&s.sfFull[i], 2);
            MbarInit(&s.sfEmpty[i], 1);
        }
        MbarInit(&s.tmemFull, 1);
        MbarInit(&s.tmemEmpty, 2 * kEpiWarps);
        s.abortFlag = 0;
        MbarInitFence();
        TmaPrefetchDesc(&tmapA);
        TmaPrefetchDesc(&tmapB);
    }
    if (warp == 3) {
        TmemAllocPair(&s.tmemBase, kTmemCols);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int acc = 0;
        s.tilePrefix[0] = 0;
        for (int g = 0; g < p.G; g++) {
            acc += s.tilePrefix[g + 1];
            s.tilePrefix[g + 1] = acc;
        }
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
        // ------------------------------------------------------------------ TMA producer (both CTAs)
        if (lane == 0) {
            const uint32_t leaderFull0 = MapToCta(SmemAddr(&s.full[0]), 0);
            uint32_t it = 0;
            for (int tile = pairId; tile < totalTiles && *abortFlag == 0; tile += pairs) {
                int g, mt, nt;
                decode(tile, g, mt, nt);
                const int rowA = p.groupOffset[g] + mt * 2 * BM + (int)cta * BM;
                const int rowB = g * p.N + nt * BN + (int)cta * BNH;
                bool ok = true;
                for (int kb = 0; kb < KB; kb++, it++) {
                    const uint32_t st = it % kStages, ph = (it / kStages) & 1;
                    if (!MbarWaitBounded(&s.empty[st], ph ^ 1, abortFlag)) {
                        ok = false;
                        break;
                    }
                    if (cta == 0) {
                        MbarExpectTx(&s.full[st], 4 * kTileBytes);  // A and weight halves of both CTAs
                    }
                    const uint32_t bar = leaderFull0 + st * (uint32_t)sizeof(uint64_t);
                    TmaLoad2DPair(s.a[st], &tmapA, bar, kb * BK, rowA);
                    TmaLoad2DPair(s.b[st], &tmapB, bar, kb * BK, rowB);
                }
                if (!ok) {
                    break;
                }
            }
        }
    } else if (warp == 2) {
        // ------------------------------------------------------------------ scale-factor producer (both CTAs)
        // One work item (tile, group of up to four K blocks) of lookahead, and a ring of two such groups of atoms with one
        // hand-shake per group, apart from the operand ring: see the one-SM kernel.
        const uint32_t leaderSfFull0 = MapToCta(SmemAddr(&s.sfFull[0]), 0);
        struct SfWords {
            uint32_t wa[4][4];
            uint32_t wb[2][4];
        };
        const bool vec = (KB & 3) == 0;
        auto fetch = [&](int tile, int kb0, SfWords &w) {
            int g, mt, nt;
            decode(tile, g, mt, nt);
            const int rowBase = p.groupOffset[g] + mt * 2 * BM + (int)cta * BM + lane;
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const int r = rowBase + 32 * j;
                if (r < p.rowsTotal) {
                    const uint32_t *src = p.aSf + (size_t)r * KB + kb0;
                    if (vec) {
                        const uint4 q = *reinterpret_cast<const uint4 *>(src);
                        w.wa[j][0] = q.x;
                        w.wa[j][1] = q.y;
                        w.wa[j][2] = q.z;
                        w.wa[j][3] = q.w;
                    } else {
#pragma unroll
                        for (int k = 0; k < 4; k++) {
                            w.wa[j][k] = kb0 + k < KB ? src[k] : kSfOne;
                        }
                    }
                } else {
#pragma unroll
                    for (int k = 0; k < 4; k++) {
                        w.wa[j][k] = kSfOne;
                    }
                }
            }
            const float *pb = p.bScale + ((size_t)g * (p.N / 128) + (size_t)nt * 2) * KB;
#pragma unroll
            for (int a = 0; a < 2; a++) {
#pragma unroll
                for (int k = 0; k < 4; k++) {
                    const float f = kb0 + k < KB ? pb[(size_t)a * KB + kb0 + k] : 1.f;
                    w.wb[a][k] = ((__float_as_uint(f) >> 23) & 0xffu) * 0x01010101u;
                }
            }
        };
        uint32_t it = 0;
        int tile = pairId, kb0 = 0;
        SfWords cur, nxt;
        bool have = tile < totalTiles;
        if (have) {
            fetch(tile, kb0, cur);
        }
        while (have && *abortFlag == 0) {
            int tileN = tile, kbN = kb0 + 4;
            if (kbN >= KB) {
                tileN = tile + pairs;
                kbN = 0;
            }
            const bool haveNext = tileN < totalTiles;
            if (haveNext) {
                fetch(tileN, kbN, nxt);
            }
            const uint32_t buf = it & 1, ph = (it >> 1) & 1;
            const bool ok = MbarWaitBounded(&s.sfEmpty[buf], ph ^ 1, abortFlag);
            if (ok) {
#pragma unroll
                for (int k = 0; k < kSfGroup; k++) {
                    if (kb0 + k >= KB) {
                        break;
                    }
                    const uint32_t slot = buf * kSfGroup + k;
                    *reinterpret_cast<uint4 *>(s.sfa[slot] + lane * 16) = make_uint4(cur.wa[0][k], cur.wa[1][k], cur.wa[2][k], cur.wa[3][k]);
#pragma unroll
                    for (int a = 0; a < 2; a++) {
                        *reinterpret_cast<uint4 *>(s.sfb[slot] + a * 512 + lane * 16) = make_uint4(cur.wb[a][k], cur.wb[a][k], cur.wb[a][k], cur.wb[a][k]);
                    }
                }
                FenceProxyAsyncShared();
                __syncwarp();
                if (lane == 0) {
                    RemoteArrive(leaderSfFull0 + buf * (uint32_t)sizeof(uint64_t));  // also the way the leader arrives on its own barrier
                }
                it++;
            }
            if (!ok) {
                break;
            }
            cur = nxt;
            tile = tileN;
            kb0 = kbN;
            have = haveNext;
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer (leader only)
        if (lane == 0 && cta == 0) {
            uint32_t it = 0, tl = 0, sg = 0;
            for (int tile = pairId; tile < totalTiles && *abortFlag == 0; tile += pairs, tl++) {
                if (!MbarWaitBounded(&s.tmemEmpty, (tl & 1) ^ 1, abortFlag)) {
                    break;
                }
                const uint32_t d = tmemBase;
                bool ok = true;
                for (int kb = 0; kb < KB; kb++, it++) {
                    const uint32_t st = it % kStages, ph = (it / kStages) & 1;
                    const uint32_t sbuf = sg & 1, slot = sbuf * kSfGroup + (kb % kSfGroup);
                    if (kb % kSfGroup == 0 && !MbarWaitBounded(&s.sfFull[sbuf], (sg >> 1) & 1, abortFlag)) {
                        ok = false;
                        break;
                    }
                    if (!MbarWaitBounded(&s.full[st], ph, abortFlag)) {
                        ok = false;
                        break;
                    }
                    TcFenceAfter();
                    const uint32_t sfa = tmemBase + kSfaCol + (kb & 1) * kSfSetCols, sfb = tmemBase + kSfbCol + (kb & 1) * kSfSetCols;
                    TmemCpSfAtomPair(sfa, SmemDescSfAtom(SmemAddr(s.sfa[slot])));
                    TmemCpSfAtomPair(sfb, SmemDescSfAtom(SmemAddr(s.sfb[slot])));
                    TmemCpSfAtomPair(sfb + 4, SmemDescSfAtom(SmemAddr(s.sfb[slot] + 512)));
                    const uint64_t aDesc = SmemDescSw128(SmemAddr(s.a[st]));
                    const uint64_t bDesc = SmemDescSw128(SmemAddr(s.b[st]));
#pragma unroll
                    for (uint32_t k = 0; k < BK / 32; k++) {
                        MmaMxF8Pair(d, aDesc + (uint64_t)(k * 2), bDesc + (uint64_t)(k * 2), InstrDescMxF8(2 * BM, BN, k), sfa | (k << 30), sfb | (k << 30),
                                    (kb > 0 || k > 0) ? 1u : 0u);
                    }
                    MmaCommitPair(&s.empty[st]);
                    if (kb % kSfGroup == kSfGroup - 1 || kb == KB - 1) {
                        MmaCommitPair(&s.sfEmpty[sbuf]);
                        sg++;
                    }
                }
                if (!ok) {
                    break;
                }
                MmaCommitPair(&s.tmemFull);
            }
        }
    } else if (warp >= 4) {
        // ------------------------------------------------------------------ epilogue (both CTAs, own 128 rows)
        const int quad = warp & 3;
        const int half = (warp - 4) >> 2;
        const int rowInTile = quad * 32 + lane;
        constexpr int NV = BN / 2;
        const int epi = p.mode & 15;
        const uint32_t leaderTmemEmpty = MapToCta(SmemAddr(&s.tmemEmpty), 0);
        uint32_t tl = 0;
        for (int tile = pairId; tile < totalTiles && *abortFlag == 0; tile += pairs, tl++) {
            int g, mt, nt;
            decode(tile, g, mt, nt);
            const int rowLocal = mt * 2 * BM + (int)cta * BM + rowInTile;
            const int row = p.groupOffset[g] + rowLocal;
            const bool valid = rowLocal < p.groupCount[g] && row < p.rowsTotal;
            if (!MbarWaitBounded(&s.tmemFull, tl & 1, abortFlag)) {
                break;
            }
            TcFenceAfter();
            const uint32_t taddr = tmemBase + ((uint32_t)(quad * 32) << 16) + half * NV;
            float v[NV];
#pragma unroll
            for (int c = 0; c < NV / 32; c++) {
                TmemLd32Issue(taddr + 32 * c, v + 32 * c);
            }
            TmemLdWait();
            TcFenceBefore();
            __syncwarp();
            if (lane == 0) {
                RemoteArrive(leaderTmemEmpty);  // the accumulator is in registers: the next tile's MMAs may overwrite it
            }
            if (!valid) {
                continue;
            }
            const int colBase = nt * BN + half * NV;
            if (epi == MF_GEMM_EPI_BF16) {
                __nv_bfloat16 *o = reinterpret_cast<__nv_bfloat16 *>(p.out) + (size_t)row * p.N + colBase;
                // Whole 32-byte sectors per store when the output allows it: half the store instructions, and no sector is
                // written in two pieces (the stores of a warp go to 32 different rows).
                if (p.wideStores) {
#pragma unroll
                    for (int j = 0; j < NV; j += 16) {
                        uint32_t pk[8];
#pragma unroll
                        for (int q = 0; q < 8; q++) {
                            const __nv_bfloat162 h2 = __floats2bfloat162_rn(v[j + 2 * q], v[j + 2 * q + 1]);
                            pk[q] = *reinterpret_cast<const uint32_t *>(&h2);
                        }
                        StGlobal32B(o + j, pk);
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < NV; j += 8) {
                        uint4 pk;
                        __nv_bfloat162 *h = reinterpret_cast<__nv_bfloat162 *>(&pk);
#pragma unroll
                        for (int q = 0; q < 4; q++) {
                            h[q] = __floats2bfloat162_rn(v[j + 2 * q], v[j + 2 * q + 1]);
                        }
                        *reinterpret_cast<uint4 *>(o + j) = pk;
                    }
                }
            } else {
#pragma unroll
                for (int q = 0; q < NV / 64; q++) {
                    float h[32];
                    float amax = 0.f;
#pragma unroll
                    for (int i = 0; i < 32; i++) {
                        h[i] = Silu(v[64 * q + i]) * v[64 * q + 32 + i];
                        amax = fmaxf(amax, fabsf(h[i]));
                    }
                    const int hcol = colBase / 2 + 32 * q;
                    if (epi == MF_GEMM_EPI_SWIGLU) {
                        __nv_bfloat16 *o = reinterpret_cast<__nv_bfloat16 *>(p.out) + (size_t)row * (p.N / 2) + hcol;
#pragma unroll
                        for (int j = 0; j < 32; j += 8) {
                            uint4 pk;
                            __nv_bfloat162 *hp = reinterpret_cast<__nv_bfloat162 *>(&pk);
#pragma unroll
                            for (int t = 0; t < 4; t++) {
                                hp[t] = __floats2bfloat162_rn(h[j + 2 * t], h[j + 2 * t + 1]);
                            }
                            *reinterpret_cast<uint4 *>(o + j) = pk;
                        }
                    } else {
                        const uint32_t e = Ue8m0Ceil(amax * (1.f / 448.f));
                        const float inv = __uint_as_float((254u - e) << 23);
                        unsigned char *o = reinterpret_cast<unsigned char *>(p.out) + (size_t)row * (p.N / 2) + hcol;
                        if (p.wideStores) {
                            uint32_t pk[8];
#pragma unroll
                            for (int t = 0; t < 8; t++) {
                                const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(h[4 * t] * inv, h[4 * t + 1] * inv), __NV_SATFINITE, __NV_E4M3);
                                const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(h[4 * t + 2] * inv, h[4 * t + 3] * inv), __NV_SATFINITE, __NV_E4M3);
                                pk[t] = lo | (hi << 16);
                            }
                            StGlobal32B(o, pk);
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; j += 16) {
                                uint4 pk;
                                unsigned short *ps = reinterpret_cast<unsigned short *>(&pk);
#pragma unroll
                                for (int t = 0; t < 8; t++) {
                                    ps[t] = __nv_cvt_float2_to_fp8x2(make_float2(h[j + 2 * t] * inv, h[j + 2 * t + 1] * inv), __NV_SATFINITE, __NV_E4M3);
                                }
                                *reinterpret_cast<uint4 *>(o + j) = pk;
                            }
                        }
                        p.outSf[(size_t)row * (p.N / 64) + hcol / 32] = (unsigned char)e;
                    }
                }
            }
        }
    }
    // ---------------------------------------------------------------------- teardown
    TcFenceBefore();
    __syncthreads();
    if (s.abortFlag != 0 && threadIdx.x == 0 && p.status != nullptr) {
        atomicCAS(p.status, 0, 3 /* pipeline wait expired */);
    }
    ClusterSync();  // neither CTA leaves (or frees TMEM) while the other may still touch its shared memory or barriers
    if (warp == 3) {
        TcFenceAfter();
        TmemDeallocPair(tmemBase, kTmemCols);
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                  const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn GetEncodeTiled2()
{
    static EncodeTiledFn fn = []() -> EncodeTiledFn {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult st;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &st) != cudaSuccess || st != cudaDriverEntryPointSuccess) {
            (void)cudaGetLastError();
            return nullptr;
        }
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    return fn;
}

bool MakeMap2(CUtensorMap *m, const void *base, uint64_t rows, uint64_t K, uint32_t boxRows)
{
    EncodeTiledFn enc = GetEncodeTiled2();
    if (enc == nullptr) {
        return false;
    }
    cuuint64_t dims[2] = {K, rows};
    cuuint64_t strides[1] = {K};
    cuuint32_t box[2] = {BK, boxRows};
    cuuint32_t estr[2] = {1, 1};
    return enc(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
               CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

// Same arguments as mf_k_moe_grouped_gemm_mx (N must be a multiple of 256). ctas: 0 = all SMs (rounded down to an even number).
extern "C" int mf_k_moe_grouped_gemm_mx_2sm(const void *a, const uint32_t *aSf, const void *b, const float *bScale, void *out, void *outSf,
                                            const int *groupOffset, const int *groupCount, int G, int rowsTotal, int N, int K, int mode, int *status,
                                            int ctas, mf_stream_t stream)
{
    const int epi = mode & 15;
    if (a == nullptr || b == nullptr || out == nullptr || aSf == nullptr || bScale == nullptr || groupOffset == nullptr || groupCount == nullptr ||
        G < 1 || G > kMaxGroups || rowsTotal < 1 || N <= 0 || K <= 0 || N % 256 != 0 || K % BK != 0 ||
        (epi != MF_GEMM_EPI_BF16 && epi != MF_GEMM_EPI_SWIGLU && epi != MF_GEMM_EPI_SWIGLU_FP8) || (epi == MF_GEMM_EPI_SWIGLU_FP8 && outSf == nullptr)) {
        return MF_K_INVALID;
    }
    if (((uintptr_t)a & 15) || ((uintptr_t)b & 15) || ((uintptr_t)out & 15) || ((uintptr_t)aSf & 15)) {
        return MF_K_INVALID;
    }
    CUtensorMap mapA, mapB;
    if (!MakeMap2(&mapA, a, (uint64_t)rowsTotal, (uint64_t)K, BM) || !MakeMap2(&mapB, b, (uint64_t)G * N, (uint64_t)K, BNH)) {
        return MF_K_LAUNCH_FAILED;
    }
    Mx2Params p;
    p.aSf = aSf;
    p.bScale = bScale;
    p.out = out;
    p.outSf = (unsigned char *)outSf;
    p.groupOffset = groupOffset;
    p.groupCount = groupCount;
    p.status = status;
    p.G = G;
    p.N = N;
    p.K = K;
    p.mode = mode;
    p.rowsTotal = rowsTotal;
    p.wideStores = ((uintptr_t)out & 31) == 0 ? 1 : 0;
    static bool attrSet = false;
    const size_t smem = sizeof(SharedStorage2) + 1024;
    if (!attrSet) {
        if (cudaFuncSetAttribute(mf_moe_grouped_gemm_mx2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
            (void)cudaGetLastError();
            return MF_K_LAUNCH_FAILED;
        }
        attrSet = true;
    }
    const int sms = mf_k_sm_count();
    if (sms < 2) {
        return MF_K_LAUNCH_FAILED;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = (cudaStream_t)stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    // The kernel is persistent with a static tile walk: every pair must be resident from the start, or the pairs of a second
    // wave would only begin when a first-wave pair has finished ALL its tiles. Not every SM can be paired (a pair needs two
    // free SMs of one cluster-scheduling group), so the number of pairs that fit at once is asked for, not assumed.
    static int maxPairs = 0;
    if (maxPairs == 0) {
        cfg.gridDim = dim3((unsigned)(sms & ~1));
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, mf_moe_grouped_gemm_mx2_kernel, &cfg) != cudaSuccess || n < 1) {
            (void)cudaGetLastError();
            return MF_K_LAUNCH_FAILED;
        }
        maxPairs = n;
    }
    int pairsWanted = (ctas > 0 && ctas < sms ? ctas : sms) / 2;
    if (pairsWanted > maxPairs) {
        pairsWanted = maxPairs;
    }
    if (pairsWanted < 1) {
        return MF_K_INVALID;
    }
    cfg.gridDim = dim3((unsigned)(2 * pairsWanted));
    if (cudaLaunchKernelEx(&cfg, mf_moe_grouped_gemm_mx2_kernel, mapA, mapB, p) != cudaSuccess) {
        (void)cudaGetLastError();
        return MF_K_LAUNCH_FAILED;
    }
    return MF_K_OK;
}
