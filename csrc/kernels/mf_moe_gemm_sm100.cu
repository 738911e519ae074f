// Grouped FP8 GEMM for the MoE expert FFN on Blackwell tensor cores (tcgen05 + TMEM + TMA), block-scaled:
//     out[g-rows, :] = (A[g-rows, :] * sa) x (B[g] * sb)^T
// A: received tokens, fp8 e4m3 with one fp32 scale per (row, 128 K-elements); B[g]: expert weights [N, K] fp8 e4m3 with one
// fp32 scale per 128x128 block. The reference library has no GEMM (MoE is only named as a use case, README.md:53 of the
// reference); the contract here is the DeepSeek-V3 block-scaled FFN of the workload definition.
//
// Mapping to the hardware, per CTA (one persistent CTA per SM, 320 threads):
//   warp 0     TMA producer: cp.async.bulk.tensor 2-D loads of a 128x128-byte A tile and a 128x128-byte B tile per K-block
//              into a 6-stage shared-memory ring (128-byte swizzle), completion on mbarriers. Loads are per-CTA, no multicast.
//   warp 1     one elected thread issues tcgen05.mma.kind::f8f6f4 (M128 N128 K32, four per K-block) into one of four
//              128-column TMEM accumulators (all 512 columns) and tcgen05.commit's to "stage free" and "partial ready" mbarriers.
//   warps 2-9  read each K-block's partial product from TMEM (tcgen05.ld 32x32b, 64 columns per thread: warps 2-5 take the
//              left half of the tile, warps 6-9 the right half), multiply by sa[row, kb] * sb[tile, kb] and add into fp32
//              registers; the four TMEM buffers let the MMAs run up to three K-blocks ahead of this promotion. After the last
//              K-block they apply the epilogue (plain, or SwiGLU on interleaved gate/up columns) and store bf16.
// Tiles are enumerated on the device from group_offset/group_count (the host does not know the routing result), n fastest so
// that concurrently running CTAs share an A tile and stream one expert's weights through L2.
// Every mbarrier wait is bounded; on expiry the CTA sets *status, all roles drain and the CTA frees its TMEM and exits.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

#include <cstdlib>

#include "mf_kernels.h"
#include "mf_sm100_ptx.cuh"

using namespace mf::sm100;

namespace {

constexpr int BM = 128, BN = 128, BK = 128;
constexpr int kStages = 6;
constexpr int kThreads = 320;
constexpr int kAccBufs = 4;                      // TMEM accumulator buffers (128 columns each)
constexpr int kEpiThreads = 256;                 // warps 2-9
constexpr int kTileBytes = BM * BK;  // fp8: 16 KiB per operand tile
constexpr int kMaxGroups = 256;
constexpr uint32_t kTmemCols = 512;

struct SharedStorage {
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

struct GemmParams {
    const float *aScale;
    const float *bScale;
    __nv_bfloat16 *out;
    const int *groupOffset;
    const int *groupCount;
    int *status;
    int G, N, K, mode, outStride, rowsTotal;
};

__device__ __forceinline__ float Silu(float x) { return x / (1.f + __expf(-x)); }

__global__ void __launch_bounds__(kThreads, 1)
mf_moe_grouped_gemm_kernel(const __grid_constant__ CUtensorMap tmapA, const __grid_constant__ CUtensorMap tmapB, const GemmParams p)
{
    extern __shared__ unsigned char smemRaw[];
    SharedStorage &s = *reinterpret_cast<SharedStorage *>((reinterpret_cast<uintptr_t>(smemRaw) + 1023) & ~(uintptr_t)1023);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int KB = p.K / BK, NT = p.N / BN;

    if (threadIdx.x == 0) {
        for (int i = 0; i < kStages; i++) {
            MbarInit(&s.full[i], 1);
            MbarInit(&s.empty[i], 1);
        }
        for (int i = 0; i < kAccBufs; i++) {
            MbarInit(&s.tmemFull[i], 1);
            MbarInit(&s.tmemEmpty[i], kEpiThreads / 32);  // one arrival per epilogue warp
        }
        s.abortFlag = 0;
        int acc = 0;
        for (int g = 0; g < p.G; g++) {
            s.tilePrefix[g] = acc;
            acc += ((p.groupCount[g] + BM - 1) / BM) * NT;
        }
        s.tilePrefix[p.G] = acc;
        MbarInitFence();
        TmaPrefetchDesc(&tmapA);
        TmaPrefetchDesc(&tmapB);
    }
    if (warp == 0) {
        TmemAlloc(&s.tmemBase, kTmemCols);
    }
    TcFenceBefore();
    __syncthreads();
    TcFenceAfter();
    const uint32_t tmemBase = s.tmemBase;
    const int totalTiles = s.tilePrefix[p.G];
    volatile int *abortFlag = &s.abortFlag;

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
            for (int tile = blockIdx.x; tile < totalTiles && *abortFlag == 0; tile += gridDim.x) {
                int g, mt, nt;
                decode(tile, g, mt, nt);
                const int rowA = p.groupOffset[g] + mt * BM;
                const int rowB = g * p.N + nt * BN;
                for (int kb = 0; kb < KB; kb++, it++) {
                    const uint32_t st = it % kStages, ph = (it / kStages) & 1;
                    if (!MbarWaitBounded(&s.empty[st], ph ^ 1, abortFlag)) {
                        break;
                    }
                    MbarExpectTx(&s.full[st], 2 * kTileBytes);
                    TmaLoad2D(s.a[st], &tmapA, &s.full[st], kb * BK, rowA);
                    TmaLoad2D(s.b[st], &tmapB, &s.full[st], kb * BK, rowB);
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = InstrDescF8(BM, BN);
            uint32_t it = 0;
            for (int tile = blockIdx.x; tile < totalTiles && *abortFlag == 0; tile += gridDim.x) {
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
                        // 32 fp8 elements = 32 bytes further along K inside the 128-byte swizzled row: +2 in 16-byte units.
                        MmaF8(d, aDesc + (uint64_t)(k * 2), bDesc + (uint64_t)(k * 2), idesc, k > 0 ? 1u : 0u);
                    }
                    MmaCommit(&s.empty[st]);      // the smem stage may be refilled once these MMAs have read it
                    MmaCommit(&s.tmemFull[buf]);  // the partial product is complete in TMEM
                }
            }
        }
    } else {
        // ------------------------------------------------------------------ promotion + epilogue (8 warps: one row, 64 columns per thread)
        const int quad = warp & 3;          // TMEM lanes this warp may touch: 32*quad .. 32*quad+31
        const int half = (warp - 2) >> 2;   // 0: tile columns [0,64), 1: [64,128)
        const int rowInTile = quad * 32 + lane;
        constexpr int HC = BN / 2;
        uint32_t it = 0;
        for (int tile = blockIdx.x; tile < totalTiles && *abortFlag == 0; tile += gridDim.x) {
            int g, mt, nt;
            decode(tile, g, mt, nt);
            const int row = p.groupOffset[g] + mt * BM + rowInTile;
            // Rows past the end of A (group tables that overrun the buffer) are never read or written.
            const bool valid = mt * BM + rowInTile < p.groupCount[g] && row < p.rowsTotal;
            const float *sa = p.aScale + (size_t)row * KB;
            const float *sb = p.bScale + ((size_t)g * NT + nt) * KB;
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
                const uint32_t taddr = tmemBase + ((uint32_t)(quad * 32) << 16) + buf * BN + half * HC;
                float v[HC];
                TmemLd32Issue(taddr, v);
                TmemLd32Issue(taddr + 32, v + 32);
                TmemLdWait();
                TcFenceBefore();
                __syncwarp();
                if (lane == 0) {
                    MbarArrive(&s.tmemEmpty[buf]);  // the warp's values are in registers: one arrival per warp keeps the barrier cheap
                }
#pragma unroll
                for (int i = 0; i < HC; i++) {
                    acc[i] = fmaf(v[i], scale, acc[i]);
                }
            }
            if (!ok) {
                break;
            }
            if (valid) {
                if ((p.mode & 15) == MF_GEMM_EPI_SWIGLU) {
                    // Each 64-column half of the tile holds 32 gate projections followed by the 32 matching up projections.
                    __nv_bfloat16 *o = p.out + (size_t)row * p.outStride + nt * (BN / 2) + half * (HC / 2);
#pragma unroll
                    for (int j = 0; j < HC / 2; j += 8) {
                        uint4 pk;
                        __nv_bfloat162 *h = reinterpret_cast<__nv_bfloat162 *>(&pk);
#pragma unroll
                        for (int q = 0; q < 4; q++) {
                            h[q] = __floats2bfloat162_rn(Silu(acc[j + 2 * q]) * acc[HC / 2 + j + 2 * q],
                                                         Silu(acc[j + 2 * q + 1]) * acc[HC / 2 + j + 2 * q + 1]);
                        }
                        *reinterpret_cast<uint4 *>(o + j) = pk;
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
    // ---------------------------------------------------------------------- teardown
    TcFenceBefore();
    __syncthreads();
    if (s.abortFlag != 0 && threadIdx.x == 0 && p.status != nullptr) {
        atomicCAS(p.status, 0, 3 /* MF_DEV_ERR_PIPELINE */);
    }
    if (warp == 0) {
        TcFenceAfter();
        TmemDealloc(tmemBase, kTmemCols);
    }
}

// ---------------------------------------------------------------------------------------------- row quantisation (bf16 → fp8, 1x128 scales)

__global__ void mf_quant_rows_fp8_kernel(const __nv_bfloat16 *__restrict__ x, unsigned char *__restrict__ q, float *__restrict__ scale, int rows, int K,
                                         const int *__restrict__ rowLimit)
{
    // One warp per (row, group of 256 elements): lanes 0-15 and 16-31 each own one 128-element block, 8 elements per lane.
    const int warpsPerBlock = blockDim.x >> 5;
    const int lane = threadIdx.x & 31;
    const int blocksPerRow = K / 128;
    const int pairsPerRow = (blocksPerRow + 1) / 2;
    const long long totalPairs = (long long)rows * pairsPerRow;
    const int limit = rowLimit != nullptr ? *rowLimit : rows;
    for (long long pr = (long long)blockIdx.x * warpsPerBlock + (threadIdx.x >> 5); pr < totalPairs; pr += (long long)gridDim.x * warpsPerBlock) {
        const int row = (int)(pr / pairsPerRow);
        if (row >= limit) {
            continue;
        }
        // With an odd number of blocks per row the upper half-warp has no block in the last pair; it walks through the same
        // instructions on a zero vector so that the full-mask shuffles below stay convergent.
        const int blk = (int)(pr % pairsPerRow) * 2 + (lane >> 4);
        const bool active = blk < blocksPerRow;
        const size_t off = (size_t)row * K + (size_t)(active ? blk : 0) * 128 + (lane & 15) * 8;
        uint4 raw = make_uint4(0u, 0u, 0u, 0u);
        if (active) {
            raw = *reinterpret_cast<const uint4 *>(x + off);
        }
        const __nv_bfloat162 *h = reinterpret_cast<const __nv_bfloat162 *>(&raw);
        float f[8];
        float amax = 0.f;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            float2 t = __bfloat1622float2(h[i]);
            f[2 * i] = t.x;
            f[2 * i + 1] = t.y;
            amax = fmaxf(amax, fmaxf(fabsf(t.x), fabsf(t.y)));
        }
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) {
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        }
        const float sc = fmaxf(amax, 1e-10f) * (1.f / 448.f);
        uint2 packed;
        unsigned short *ps = reinterpret_cast<unsigned short *>(&packed);
#pragma unroll
        for (int i = 0; i < 4; i++) {
            ps[i] = __nv_cvt_float2_to_fp8x2(make_float2(f[2 * i] / sc, f[2 * i + 1] / sc), __NV_SATFINITE, __NV_E4M3);
        }
        if (active) {
            *reinterpret_cast<uint2 *>(q + off) = packed;
            if ((lane & 15) == 0) {
                scale[(size_t)row * blocksPerRow + blk] = sc;
            }
        }
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

// [rows, K] uint8 row-major, boxes of 128 (K) x 128 (rows), 128-byte swizzle.
bool MakeMap(CUtensorMap *m, const void *base, uint64_t rows, uint64_t K)
{
    EncodeTiledFn enc = GetEncodeTiled();
    if (enc == nullptr) {
        return false;
    }
    cuuint64_t dims[2] = {K, rows};
    cuuint64_t strides[1] = {K};
    cuuint32_t box[2] = {BK, BM};
    cuuint32_t estr[2] = {1, 1};
    return enc(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
               CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

extern "C" int mf_k_moe_grouped_gemm(const void *a, const float *aScale, const void *b, const float *bScale, void *out, const int *groupOffset,
                                     const int *groupCount, int G, int rowsTotal, int N, int K, int mode, int *status, int ctas, mf_stream_t stream)
{
    if (a == nullptr || b == nullptr || out == nullptr || aScale == nullptr || bScale == nullptr || groupOffset == nullptr || groupCount == nullptr ||
        G < 1 || G > kMaxGroups || rowsTotal < 1 || N % BN != 0 || K % BK != 0 || N <= 0 || K <= 0) {
        return MF_K_INVALID;
    }
    if (((uintptr_t)a & 15) || ((uintptr_t)b & 15) || ((uintptr_t)out & 15)) {
        return MF_K_INVALID;  // TMA base addresses and the 16-byte epilogue stores need 16-byte alignment
    }
    CUtensorMap mapA, mapB;
    if (!MakeMap(&mapA, a, (uint64_t)rowsTotal, (uint64_t)K) || !MakeMap(&mapB, b, (uint64_t)G * N, (uint64_t)K)) {
        return MF_K_LAUNCH_FAILED;
    }
    if (ctas < 0) {
        ctas = 0;
    }
    GemmParams p;
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
    p.rowsTotal = rowsTotal;
    static bool attrSet = false;
    const size_t smem = sizeof(SharedStorage) + 1024;
    if (!attrSet) {
        if (cudaFuncSetAttribute(mf_moe_grouped_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
            (void)cudaGetLastError();
            return MF_K_LAUNCH_FAILED;
        }
        attrSet = true;
    }
    int sms = mf_k_sm_count();
    if (sms <= 0) {
        return MF_K_LAUNCH_FAILED;
    }
    int grid = ctas > 0 && ctas < sms ? ctas : sms;
    mf_moe_grouped_gemm_kernel<<<grid, kThreads, smem, (cudaStream_t)stream>>>(mapA, mapB, p);
    return cudaGetLastError() == cudaSuccess ? MF_K_OK : MF_K_LAUNCH_FAILED;
}

extern "C" int mf_k_quant_rows_fp8(const void *x, void *q, float *scale, int rows, int K, const int *rowLimit, mf_stream_t stream)
{
    if (x == nullptr || q == nullptr || scale == nullptr || rows < 1 || K % 128 != 0) {
        return MF_K_INVALID;
    }
    long long pairs = (long long)rows * ((K / 128 + 1) / 2);
    long long blocks = (pairs + 7) / 8;
    if (blocks > 148 * 16) {
        blocks = 148 * 16;
    }
    mf_quant_rows_fp8_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16 *)x, (unsigned char *)q, scale, rows, K, rowLimit);
    return cudaGetLastError() == cudaSuccess ? MF_K_OK : MF_K_LAUNCH_FAILED;
}
