// Grouped FP8 GEMM for the MoE expert FFN on Blackwell tensor cores with HARDWARE block scaling
// (tcgen05.mma.kind::mxf8f6f4.block_scale): the whole K reduction of a tile accumulates in TMEM and the epilogue runs once
// per tile, instead of promoting every 128-wide K block through registers.
//     out[g-rows, :] = (A[g-rows, :] * 2^ea) x (B[g] * 2^eb)^T
// A: received tokens, e4m3, one power-of-two scale (UE8M0 byte) per (row, 32 K-elements) packed four to a 32-bit word per
// 128-element K block; B[g]: expert weights [N, K] e4m3 with one power-of-two fp32 scale per 128x128 block. The reference
// library has no GEMM (MoE is only named as a use case, README.md:53 of the reference); the contract is the DeepSeek-V3
// block-scaled FFN of the workload definition with scales rounded up to powers of two, which is what the tensor core applies.
//
// Mapping to the hardware, per CTA (one persistent CTA per SM, 384 threads):
//   warp 0      TMA producer: cp.async.bulk.tensor 2-D loads of a 128x128-byte A tile and a BNx128-byte B tile per K block into
//               a shared-memory ring (128-byte swizzle), completion on mbarriers. Per-CTA loads of local memory, no multicast.
//   warp 2      scale-factor producer: gathers the 128 A-row scale words and the weight-block scales of the K block and lays
//               them out in shared memory in the 32x16-byte atoms that tcgen05.cp copies to TMEM.
//   warp 1      one thread copies the scale atoms to TMEM (tcgen05.cp) and issues four tcgen05.mma (M128, N = BN, K32) per K
//               block; tcgen05.commit hands the smem stage back and, after the last K block, publishes the accumulator.
//   warps 4-11  epilogue: tcgen05.ld the finished accumulator (one row, BN/2 columns per thread), release TMEM at once, then
//               either store bf16, or apply SwiGLU on interleaved gate/up columns and quantise the result to e4m3 with one
//               UE8M0 scale per 32 outputs, which is exactly the A operand format of the second GEMM (no separate
//               quantisation kernel, no bf16 round trip of the intermediate).
// BN = 256 (one accumulator of 256 TMEM columns, 4-stage ring) for large row counts; BN = 128 (two accumulators, 6-stage ring)
// when there are few rows per expert and the kernel streams weights (more, smaller tiles balance the 148 SMs better);
// BN = 224 (two accumulators of 224 columns, 4-stage ring) for the plain bf16 epilogue when N is a multiple of 224: nearly
// the operand reuse of the 256-wide tile, and the epilogue of one tile runs under the MMAs of the next, which matters when K
// is short (the second FFN GEMM: N = 7168 = 32 x 224, K = 2048).
// Every mbarrier wait is bounded; on expiry the CTA sets *status, all roles drain and the CTA frees its TMEM and exits.
// Gated form (mf_k_moe_grouped_gemm_mx_gated): the rows of A are being stored by other GPUs (the MoE dispatch of the peers)
// while this kernel runs. The two warps that read A — the TMA producer and the scale-factor producer — start a tile only when
// the arrival counter of its 128 rows is complete (acquire load of system scope, then a proxy fence before the TMA reads);
// the scale-factor producer looks one tile ahead without blocking so that a tile that is late does not stall the one in flight.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

#include <cstdlib>

#include "mf_kernels.h"
#include "mf_sm100_ptx.cuh"

using namespace mf::sm100;

namespace {

constexpr int BM = 128, BK = 128;
constexpr int kThreads = 384;
constexpr int kEpiWarps = 8;
constexpr int kMaxGroups = 256;
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kSfOne = 0x7f7f7f7fu;  // four UE8M0 bytes of value 1.0

template <int BN>
struct Cfg {
    static constexpr int kStages = BN == 128 ? 6 : 4;
    static constexpr int kAccBufs = BN == 256 ? 1 : 2;
    static constexpr int kAtomsB = (BN + 127) / 128;
    static constexpr int kSfbWords = BN % 128 == 0 ? 1 : 4;  // distinct weight-scale words per 128-column atom
    static constexpr int kATile = BM * BK;  // bytes (fp8)
    static constexpr int kBTile = BN * BK;
    // TMEM columns: the accumulators come first, then four columns of A scale factors, then four per 128 columns of B.
    static constexpr uint32_t kSfaCol = kAccBufs * BN;
    static constexpr uint32_t kSfbCol = kSfaCol + 4;
    static_assert(kSfbCol + 4 * kAtomsB <= kTmemCols, "accumulators and scale factors must fit the 512 TMEM columns");
    static_assert(kBTile % 1024 == 0, "stages of the B ring must stay 1024-byte aligned for the 128-byte swizzle");
};

template <int BN>
struct SharedStorage {
    alignas(1024) unsigned char a[Cfg<BN>::kStages][Cfg<BN>::kATile];
    alignas(1024) unsigned char b[Cfg<BN>::kStages][Cfg<BN>::kBTile];
    alignas(128) unsigned char sfa[Cfg<BN>::kStages][512];
    alignas(128) unsigned char sfb[Cfg<BN>::kStages][512 * Cfg<BN>::kAtomsB];
    uint64_t full[Cfg<BN>::kStages];
    uint64_t empty[Cfg<BN>::kStages];
    uint64_t tmemFull[2];
    uint64_t tmemEmpty[2];
    uint32_t tmemBase;
    int abortFlag;  // 0 running, 1 a pipeline wait expired, 2 an arrival wait expired
    int gated;
    int tilePrefix[kMaxGroups + 1];
};

struct MxParams {
    const uint32_t *aSf;
    const float *bScale;
    void *out;
    unsigned char *outSf;
    const int *groupOffset;
    const int *groupCount;
    int *status;
    int G, N, K, mode, rowsTotal;
    const int *arrive;  // optional: rows landed per 128-row tile of A
    uint64_t waitNs;
    int wideStores;  // out is 32-byte aligned: the epilogue stores whole sectors
    int bPacked;     // weights are stored as [G][N/32][K/128][32][128] and tmapB is the 4-D map of that layout
};

__device__ __forceinline__ int LdAcquireSys(const int *p)
{
    int v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Spins until *ctr >= need; what the senders stored before they counted their rows is visible afterwards. Bounded: on expiry
// the CTA-wide abort flag is raised and every role drains.
__device__ __forceinline__ bool ArrivalWait(const int *ctr, int need, volatile int *abortFlag, uint64_t limitNs)
{
    if (LdAcquireSys(ctr) >= need) {
        return true;
    }
    const uint64_t t0 = GlobalTimerNs();
    for (uint32_t i = 0; i < (1u << 24); i++) {
        if (LdAcquireSys(ctr) >= need) {
            return true;
        }
        if ((i & 15u) == 15u) {
            if (*abortFlag != 0) {
                return false;
            }
            if (GlobalTimerNs() - t0 > limitNs) {
                break;
            }
        }
    }
    *abortFlag = 2;
    return false;
}

__device__ __forceinline__ float Silu(float x) { return x / (1.f + __expf(-x)); }

// UE8M0 byte (biased exponent) of the smallest power of two >= t, clamped to [1, 253] so that its reciprocal is a normal float.
__device__ __forceinline__ uint32_t Ue8m0Ceil(float t)
{
    const uint32_t bits = __float_as_uint(t);
    uint32_t e = ((bits >> 23) & 0xffu) + ((bits & 0x7fffffu) != 0u ? 1u : 0u);
    return e < 1u ? 1u : (e > 253u ? 253u : e);
}

template <int BN>
__global__ void __launch_bounds__(kThreads, 1)
mf_moe_grouped_gemm_mx_kernel(const __grid_constant__ CUtensorMap tmapA, const __grid_constant__ CUtensorMap tmapB, const MxParams p)
{
    using C = Cfg<BN>;
    extern __shared__ unsigned char smemRaw[];
    SharedStorage<BN> &s = *reinterpret_cast<SharedStorage<BN> *>((reinterpret_cast<uintptr_t>(smemRaw) + 1023) & ~(uintptr_t)1023);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int KB = p.K / BK, NT = p.N / BN;

    for (int g = threadIdx.x; g < p.G; g += kThreads) {
        s.tilePrefix[g + 1] = ((p.groupCount[g] + BM - 1) / BM) * NT;
    }
    if (threadIdx.x == 0) {
        for (int i = 0; i < C::kStages; i++) {
            MbarInit(&s.full[i], 2);  // TMA thread (with the byte count) + scale-factor warp
            MbarInit(&s.empty[i], 1);
        }
        for (int i = 0; i < 2; i++) {
            MbarInit(&s.tmemFull[i], 1);
            MbarInit(&s.tmemEmpty[i], kEpiWarps);
        }
        s.abortFlag = 0;
        s.gated = p.arrive != nullptr && (p.status == nullptr || *(volatile int *)p.status == 0) ? 1 : 0;
        MbarInitFence();
        TmaPrefetchDesc(&tmapA);
        TmaPrefetchDesc(&tmapB);
    }
    if (warp == 3) {
        TmemAlloc(&s.tmemBase, kTmemCols);
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
    TcFenceAfter();
    const uint32_t tmemBase = s.tmemBase;
    const int totalTiles = s.tilePrefix[p.G];
    volatile int *abortFlag = &s.abortFlag;
    const bool gated = s.gated != 0;

    auto decode = [&](int tile, int &g, int &mt, int &nt) {
        int lo = 0, hi = p.G;  // last group whose first tile is <= tile (empty groups share a prefix value: take the last)
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
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            uint32_t it = 0;
            int lastGate = -1;
            for (int tile = blockIdx.x; tile < totalTiles && *abortFlag == 0; tile += gridDim.x) {
                int g, mt, nt;
                decode(tile, g, mt, nt);
                const int rowA = p.groupOffset[g] + mt * BM;
                const int rowB = g * p.N + nt * BN;
                if (gated && (rowA >> 7) != lastGate) {
                    if (!ArrivalWait(p.arrive + (rowA >> 7), min(BM, p.groupCount[g] - mt * BM), abortFlag, p.waitNs)) {
                        break;
                    }
                    FenceProxyAsyncGlobal();  // the rows were stored through the generic proxy (by other GPUs); TMA reads them
                    lastGate = rowA >> 7;
                }
                for (int kb = 0; kb < KB; kb++, it++) {
                    const uint32_t st = it % C::kStages, ph = (it / C::kStages) & 1;
                    if (!MbarWaitBounded(&s.empty[st], ph ^ 1, abortFlag)) {
                        break;
                    }
                    MbarExpectTx(&s.full[st], C::kATile + C::kBTile);
                    TmaLoad2D(s.a[st], &tmapA, &s.full[st], kb * BK, rowA);
                    if (p.bPacked) {
                        TmaLoad4D(s.b[st], &tmapB, &s.full[st], 0, 0, kb, rowB / 32);  // BN/32 blocks of 32 rows, 4 KiB each
                    } else {
                        TmaLoad2D(s.b[st], &tmapB, &s.full[st], kb * BK, rowB);
                    }
                }
            }
        }
    } else if (warp == 2) {
        // ------------------------------------------------------------------ scale-factor producer
        // Work item = (tile, group of up to four K blocks). The scale words of item i+1 are requested from global memory before
        // item i is laid out, so their latency (the A scales are read once and come from DRAM) is hidden behind the stage
        // hand-shakes instead of being paid once per group on the path that feeds the MMAs.
        struct SfWords {
            uint32_t wa[4][4];
            uint32_t wb[C::kAtomsB][C::kSfbWords][4];
        };
        const bool vec = (KB & 3) == 0;
        auto fetch = [&](int tile, int kb0, SfWords &w) {
            int g, mt, nt;
            decode(tile, g, mt, nt);
            const int rowBase = p.groupOffset[g] + mt * BM + lane;
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
            // Word j of atom a holds the scale of tile columns a*128 + 32*j .. +31, which lie inside ONE 128-column weight
            // block (tiles start at multiples of 32); with BN = 224 a tile spans up to three blocks.
#pragma unroll
            for (int a = 0; a < C::kAtomsB; a++) {
#pragma unroll
                for (int j = 0; j < C::kSfbWords; j++) {
                    const int cin = a * 128 + 32 * j;
                    const float *pb = p.bScale + ((size_t)g * (p.N / 128) + (size_t)((nt * BN + cin) / 128)) * KB;
#pragma unroll
                    for (int k = 0; k < 4; k++) {
                        const float f = (cin < BN && kb0 + k < KB) ? pb[kb0 + k] : 1.f;
                        w.wb[a][j][k] = ((__float_as_uint(f) >> 23) & 0xffu) * 0x01010101u;
                    }
                }
            }
        };
        // Have the 128 rows of the tile landed? Lane 0 asks (waiting if `block`), the warp shares the answer.
        auto gate = [&](int tile, bool block) -> bool {
            int ok = 1;
            if (lane == 0) {
                int g, mt, nt;
                decode(tile, g, mt, nt);
                const int row0 = p.groupOffset[g] + mt * BM;
                const int need = min(BM, p.groupCount[g] - mt * BM);
                const int *ctr = p.arrive + (row0 >> 7);
                ok = block ? (ArrivalWait(ctr, need, abortFlag, p.waitNs) ? 1 : 0) : (LdAcquireSys(ctr) >= need ? 1 : 0);
            }
            ok = __shfl_sync(0xffffffffu, ok, 0);
            __syncwarp();
            return ok != 0;
        };
        uint32_t it = 0;
        int tile = blockIdx.x, kb0 = 0;
        SfWords cur, nxt;
        bool have = tile < totalTiles;
        if (have) {
            if (gated && !gate(tile, true)) {
                have = false;
            } else {
                fetch(tile, kb0, cur);
            }
        }
        while (have && *abortFlag == 0) {
            int tileN = tile, kbN = kb0 + 4;
            if (kbN >= KB) {
                tileN = tile + (int)gridDim.x;
                kbN = 0;
            }
            const bool haveNext = tileN < totalTiles;
            bool fetched = false;
            if (haveNext && (!gated || kbN != 0 || gate(tileN, false))) {
                fetch(tileN, kbN, nxt);
                fetched = true;
            }
            bool ok = true;
#pragma unroll
            for (int k = 0; k < 4; k++) {
                if (kb0 + k >= KB) {
                    break;
                }
                const uint32_t st = it % C::kStages, ph = (it / C::kStages) & 1;
                if (!MbarWaitBounded(&s.empty[st], ph ^ 1, abortFlag)) {
                    ok = false;
                    break;
                }
                *reinterpret_cast<uint4 *>(s.sfa[st] + lane * 16) = make_uint4(cur.wa[0][k], cur.wa[1][k], cur.wa[2][k], cur.wa[3][k]);
#pragma unroll
                for (int a = 0; a < C::kAtomsB; a++) {
                    // with one word per atom (the atom lies in one weight block) all four lanes-of-32 groups share it
                    *reinterpret_cast<uint4 *>(s.sfb[st] + a * 512 + lane * 16) =
                        make_uint4(cur.wb[a][0][k], cur.wb[a][1 % C::kSfbWords][k], cur.wb[a][2 % C::kSfbWords][k], cur.wb[a][3 % C::kSfbWords][k]);
                }
                FenceProxyAsyncShared();
                __syncwarp();
                if (lane == 0) {
                    MbarArrive(&s.full[st]);
                }
                it++;
            }
            if (!ok) {
                break;
            }
            if (haveNext && !fetched) {
                if (!gate(tileN, true)) {
                    break;
                }
                fetch(tileN, kbN, nxt);
            }
            cur = nxt;
            tile = tileN;
            kb0 = kbN;
            have = haveNext;
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            uint32_t it = 0, tl = 0;
            for (int tile = blockIdx.x; tile < totalTiles && *abortFlag == 0; tile += gridDim.x, tl++) {
                const uint32_t buf = tl % C::kAccBufs, bph = (tl / C::kAccBufs) & 1;
                if (!MbarWaitBounded(&s.tmemEmpty[buf], bph ^ 1, abortFlag)) {
                    break;
                }
                const uint32_t d = tmemBase + buf * BN;
                bool ok = true;
                for (int kb = 0; kb < KB; kb++, it++) {
                    const uint32_t st = it % C::kStages, ph = (it / C::kStages) & 1;
                    if (!MbarWaitBounded(&s.full[st], ph, abortFlag)) {
                        ok = false;
                        break;
                    }
                    TcFenceAfter();
                    TmemCpSfAtom(tmemBase + C::kSfaCol, SmemDescSfAtom(SmemAddr(s.sfa[st])));
#pragma unroll
                    for (int a = 0; a < C::kAtomsB; a++) {
                        TmemCpSfAtom(tmemBase + C::kSfbCol + 4 * a, SmemDescSfAtom(SmemAddr(s.sfb[st] + a * 512)));
                    }
                    const uint64_t aDesc = SmemDescSw128(SmemAddr(s.a[st]));
                    const uint64_t bDesc = SmemDescSw128(SmemAddr(s.b[st]));
#pragma unroll
                    for (uint32_t k = 0; k < BK / 32; k++) {
                        // 32 fp8 elements = 32 bytes further along K inside the 128-byte swizzled row: +2 in 16-byte units. The byte of
                        // the scale-factor columns that belongs to this K step rides in the top two address bits and the descriptor.
                        MmaMxF8(d, aDesc + (uint64_t)(k * 2), bDesc + (uint64_t)(k * 2), InstrDescMxF8(BM, BN, k), (tmemBase + C::kSfaCol) | (k << 30),
                                (tmemBase + C::kSfbCol) | (k << 30), (kb > 0 || k > 0) ? 1u : 0u);
                    }
                    MmaCommit(&s.empty[st]);  // the stage (operands and scale atoms) may be refilled once these operations have read it
                }
                if (!ok) {
                    break;
                }
                MmaCommit(&s.tmemFull[buf]);
            }
        }
    } else if (warp >= 4) {
        // ------------------------------------------------------------------ epilogue (8 warps: one row, BN/2 columns per thread)
        const int quad = warp & 3;         // TMEM lanes this warp may touch: 32*quad .. 32*quad+31
        const int half = (warp - 4) >> 2;  // 0: tile columns [0, BN/2), 1: [BN/2, BN)
        const int rowInTile = quad * 32 + lane;
        constexpr int NV = BN / 2;
        const int epi = p.mode & 15;
        uint32_t tl = 0;
        for (int tile = blockIdx.x; tile < totalTiles && *abortFlag == 0; tile += gridDim.x, tl++) {
            int g, mt, nt;
            decode(tile, g, mt, nt);
            const uint32_t buf = tl % C::kAccBufs, bph = (tl / C::kAccBufs) & 1;
            const int row = p.groupOffset[g] + mt * BM + rowInTile;
            const bool valid = mt * BM + rowInTile < p.groupCount[g] && row < p.rowsTotal;
            if (!MbarWaitBounded(&s.tmemFull[buf], bph, abortFlag)) {
                break;
            }
            TcFenceAfter();
            const uint32_t taddr = tmemBase + ((uint32_t)(quad * 32) << 16) + buf * BN + half * NV;
            float v[NV];
#pragma unroll
            for (int c = 0; c < NV / 32; c++) {
                TmemLd32Issue(taddr + 32 * c, v + 32 * c);
            }
            if (NV % 32 != 0) {
                TmemLd16Issue(taddr + (NV / 32) * 32, v + (NV / 32) * 32);  // BN = 224: 112 columns per thread = 3 x 32 + 16
            }
            TmemLdWait();
            TcFenceBefore();
            __syncwarp();
            if (lane == 0) {
                MbarArrive(&s.tmemEmpty[buf]);  // the accumulator is in registers: the next tile's MMAs may overwrite it
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
            } else if (BN % 128 == 0) {
                // Every 64 columns hold 32 gate projections followed by the 32 matching up projections.
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
        atomicCAS(p.status, 0, s.abortFlag == 2 ? MF_K_GEMM_ARRIVAL_EXPIRED : MF_K_GEMM_PIPELINE_EXPIRED);
    }
    if (warp == 3) {
        TcFenceAfter();
        TmemDealloc(tmemBase, kTmemCols);
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                  const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn GetEncodeTiled()
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

// [rows, K] uint8 row-major, boxes of 128 (K) x boxRows, 128-byte swizzle.
bool MakeMap(CUtensorMap *m, const void *base, uint64_t rows, uint64_t K, uint32_t boxRows)
{
    EncodeTiledFn enc = GetEncodeTiled();
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

// Packed weights: [rows/32][K/128][32][128] bytes seen as a 4-D tensor {128, 32, K/128, rows/32}; a box is {128, 32, 1, boxRows/32},
// which lands in shared memory as boxRows consecutive 128-byte rows, exactly like the 2-D box of the row-major layout.
bool MakeMapPacked(CUtensorMap *m, const void *base, uint64_t rows, uint64_t K, uint32_t boxRows)
{
    EncodeTiledFn enc = GetEncodeTiled();
    if (enc == nullptr) {
        return false;
    }
    const uint64_t KB = K / BK;
    cuuint64_t dims[4] = {BK, 32, KB, rows / 32};
    cuuint64_t strides[3] = {BK, 32 * BK, KB * 32 * BK};
    cuuint32_t box[4] = {BK, 32, 1, boxRows / 32};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    return enc(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
               CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int BN>
int Launch(const CUtensorMap &mapA, const CUtensorMap &mapB, const MxParams &p, int ctas, cudaStream_t stream)
{
    static bool attrSet = false;
    const size_t smem = sizeof(SharedStorage<BN>) + 1024;
    if (!attrSet) {
        if (cudaFuncSetAttribute(mf_moe_grouped_gemm_mx_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
            (void)cudaGetLastError();
            return MF_K_LAUNCH_FAILED;
        }
        attrSet = true;
    }
    const int sms = mf_k_sm_count();
    if (sms <= 0) {
        return MF_K_LAUNCH_FAILED;
    }
    const int grid = ctas > 0 && ctas < sms ? ctas : sms;
    mf_moe_grouped_gemm_mx_kernel<BN><<<grid, kThreads, smem, stream>>>(mapA, mapB, p);
    return cudaGetLastError() == cudaSuccess ? MF_K_OK : MF_K_LAUNCH_FAILED;
}

int GemmMx(const void *a, const uint32_t *aSf, const void *b, const float *bScale, void *out, void *outSf, const int *groupOffset,
           const int *groupCount, int G, int rowsTotal, int N, int K, int mode, int tileN, const int *arrive, uint64_t waitNs, int *status, int ctas,
           mf_stream_t stream)
{
    const int epi = mode & 15;
    const bool packed = (mode & MF_GEMM_B_PACKED) != 0;
    if (tileN == 512) {
        if (arrive != nullptr || packed) {
            return MF_K_INVALID;
        }
        return mf_k_moe_grouped_gemm_mx_2sm(a, aSf, b, bScale, out, outSf, groupOffset, groupCount, G, rowsTotal, N, K, mode, status, ctas, stream);
    }
    if (a == nullptr || b == nullptr || out == nullptr || aSf == nullptr || bScale == nullptr || groupOffset == nullptr || groupCount == nullptr ||
        G < 1 || G > kMaxGroups || rowsTotal < 1 || N <= 0 || K <= 0 || N % 128 != 0 || K % BK != 0 ||
        (epi != MF_GEMM_EPI_BF16 && epi != MF_GEMM_EPI_SWIGLU && epi != MF_GEMM_EPI_SWIGLU_FP8) || (epi == MF_GEMM_EPI_SWIGLU_FP8 && outSf == nullptr) ||
        (tileN != 0 && tileN != 128 && tileN != 224 && tileN != 256)) {
        return MF_K_INVALID;
    }
    if (((uintptr_t)a & 15) || ((uintptr_t)b & 15) || ((uintptr_t)out & 15) || ((uintptr_t)aSf & 15)) {
        return MF_K_INVALID;  // TMA base addresses, the 16-byte scale-word loads and the 16-byte epilogue stores need 16-byte alignment
    }
    if (tileN == 0) {
        // Wide tiles when every SM gets at least two of them even so; otherwise more, narrower tiles balance better. The plain
        // bf16 epilogue prefers the double-buffered 224-column tile where N allows it.
        const long long mTiles = (rowsTotal + BM - 1) / BM;
        static const bool auto224 = []() {
            const char *e = getenv("MF_GEMM_TILE224");
            return e != nullptr && e[0] == '1';
        }();
        // Measured on the second FFN GEMM (N 7168, K 2048): with at most one m-tile per expert (decode) the 224-column tile is 4 %
        // faster than the 256-column one, with 1024 rows per expert it is 6 % slower, so it is chosen for the former only
        // (MF_GEMM_TILE224=1 forces it wherever it applies).
        const bool fewRows = mTiles <= (long long)G;
        if ((auto224 || fewRows) && epi == MF_GEMM_EPI_BF16 && N % 224 == 0 && mTiles * (N / 224) >= 2LL * 148) {
            tileN = 224;
        } else {
            tileN = (N % 256 == 0 && mTiles * (N / 256) >= 2LL * 148) ? 256 : 128;
        }
    }
    if ((tileN == 256 && N % 256 != 0) || (tileN == 224 && (N % 224 != 0 || epi != MF_GEMM_EPI_BF16))) {
        return MF_K_INVALID;
    }
    CUtensorMap mapA, mapB;
    if (!MakeMap(&mapA, a, (uint64_t)rowsTotal, (uint64_t)K, BM) ||
        !(packed ? MakeMapPacked(&mapB, b, (uint64_t)G * N, (uint64_t)K, (uint32_t)tileN) : MakeMap(&mapB, b, (uint64_t)G * N, (uint64_t)K, (uint32_t)tileN))) {
        return MF_K_LAUNCH_FAILED;
    }
    MxParams p;
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
    p.arrive = arrive;
    p.wideStores = ((uintptr_t)out & 31) == 0 ? 1 : 0;
    p.bPacked = packed ? 1 : 0;
    // Shorter than the 2 s limit of the pipeline waits, so that a tile that never arrives is reported as such.
    p.waitNs = (waitNs == 0 || waitNs > 1500000000ull) ? 1500000000ull : waitNs;
    if (tileN == 224) {
        return Launch<224>(mapA, mapB, p, ctas, (cudaStream_t)stream);
    }
    return tileN == 256 ? Launch<256>(mapA, mapB, p, ctas, (cudaStream_t)stream) : Launch<128>(mapA, mapB, p, ctas, (cudaStream_t)stream);
}

}  // namespace

extern "C" int mf_k_moe_grouped_gemm_mx(const void *a, const uint32_t *aSf, const void *b, const float *bScale, void *out, void *outSf,
                                        const int *groupOffset, const int *groupCount, int G, int rowsTotal, int N, int K, int mode, int tileN,
                                        int *status, int ctas, mf_stream_t stream)
{
    return GemmMx(a, aSf, b, bScale, out, outSf, groupOffset, groupCount, G, rowsTotal, N, K, mode, tileN, nullptr, 0, status, ctas, stream);
}

extern "C" int mf_k_moe_grouped_gemm_mx_gated(const void *a, const uint32_t *aSf, const void *b, const float *bScale, void *out, void *outSf,
                                              const int *groupOffset, const int *groupCount, int G, int rowsTotal, int N, int K, int mode, int tileN,
                                              const int *arrive, uint64_t waitNs, int *status, int ctas, mf_stream_t stream)
{
    if (arrive == nullptr) {
        return MF_K_INVALID;
    }
    return GemmMx(a, aSf, b, bScale, out, outSf, groupOffset, groupCount, G, rowsTotal, N, K, mode, tileN, arrive, waitNs, status, ctas, stream);
}
