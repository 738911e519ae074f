// RL weight reshard: training layout (one flat bf16 parameter vector, evenly sharded over R ranks — the FSDP layout) →
// inference layout of one rank (its tensor-parallel sub-block of every parameter), optionally cast to e4m3 with 128x128
// block scales, as ONE gather kernel that pulls exactly the bytes this rank needs from the owners' shards over NVLink.
// The reference names parameter resharding for reinforcement learning only as a use case of its global address space
// (README.md:53 of the reference); the all-gather-then-slice it replaces moves R x more data.
//
// The host describes the destination as a table of parameter sub-blocks (origin + shape inside the full parameter, where
// the parameter sits in the flat vector, where the sub-block goes). The kernel enumerates 128x128 tiles over the table
// (binary search of a prefix of tile counts), and for each tile: computes, per 16-byte vector, which rank's shard holds it
// (shards are multiples of 8 elements, so a vector never straddles two ranks), loads it from that rank's heap, and either
// stores it (bf16) or reduces the tile's absolute maximum, scales and converts to e4m3 (one fp32 scale per tile).
// A barrier over all ranks opens the kernel (every shard is final) and closes it (nobody reuses its shard while it is read).
#include <cooperative_groups.h>
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

#include "mf/device/mf_shm_device.cuh"
#include "mf_kernels.h"

namespace cg = cooperative_groups;

namespace {

constexpr int kThreads = 512;
constexpr int kTile = 128;           // quantisation block edge and tile height
constexpr int kTileCols = 256;       // tile width: a warp reads 512 contiguous bytes of a row (two quantisation blocks)
constexpr int kVecPerRow = kTileCols / 8;
constexpr int kVecPerThread = (kTile * kTileCols / 8) / kThreads;  // 8

__global__ void __launch_bounds__(kThreads, 2)
mf_reshard_kernel(const mf_reshard_args_t *__restrict__ args, uint32_t channel, uint64_t epoch, uint64_t timeoutNs)
{
    cg::grid_group grid = cg::this_grid();
    const mf_reshard_args_t a = args[blockIdx.y];
    const MfDeviceMeta *m = reinterpret_cast<const MfDeviceMeta *>(a.meta);
    __shared__ float warpMax[2][kThreads / 32];  // per quantisation block of the tile, per warp
    __shared__ int abortFlag;
    if (mf_check_bounds_enabled(m) && !mf_shm_in_own_window(m, a.srcShard, a.shardElems * 2)) {
        if (threadIdx.x == 0 && a.status != nullptr) {
            atomicCAS(a.status, 0, MF_DEV_ERR_BOUNDS);
        }
        return;
    }

    if (blockIdx.x == 0) {
        int rc = mf_barrier_cta(m, channel, 0, 2 * epoch - 1, timeoutNs);
        if (rc != MF_DEV_OK && threadIdx.x == 0 && a.status != nullptr) {
            atomicCAS(a.status, 0, rc);
        }
    }
    grid.sync();
    if (threadIdx.x == 0) {
        abortFlag = a.status != nullptr ? *(volatile int *)a.status : 0;
    }
    __syncthreads();
    const bool dead = abortFlag != 0;

    // rank 0's copy of the shard buffer: rank r's is r * symmetricSize further
    const char *shard0 = reinterpret_cast<const char *>(a.srcShard) - (uint64_t)m->rankId * m->symmetricSize;
    if (!dead) {
        // Blocked distribution: every CTA walks a contiguous run of tiles (same rows, neighbouring columns, then the next rows),
        // so its reads stay inside a few pages of one owner at a time instead of hopping across all peers' shards.
        const uint32_t perCta = (a.totalTiles + gridDim.x - 1) / gridDim.x;
        const uint32_t tileEnd = min(a.totalTiles, (blockIdx.x + 1) * perCta);
        for (uint32_t tile = blockIdx.x * perCta; tile < tileEnd; tile++) {
            uint32_t lo = 0, hi = a.ndesc;
            while (hi - lo > 1) {
                const uint32_t mid = (lo + hi) >> 1;
                if (a.descs[mid].tileStart <= tile) {
                    lo = mid;
                } else {
                    hi = mid;
                }
            }
            const mf_reshard_desc_t &d = a.descs[lo];
            const uint32_t nrows = d.nrows, ncols = d.ncols, colsFull = d.colsFull;
            const uint32_t tilesPerRow = (ncols + kTileCols - 1) / kTileCols;
            const uint32_t local = tile - d.tileStart;
            const uint32_t tr = local / tilesPerRow, tc = local % tilesPerRow;
            const uint32_t rowBase = tr * kTile, colBase = tc * kTileCols;
            // A warp reads one row segment of 512 bytes per trip: lane l owns columns colBase + 8l .. +7 of rows
            // rowBase + warp, + 16, + 32, ... (16 warps, 8 trips).
            const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
            const uint32_t c = colBase + lane * 8;
            const bool colOk = c < ncols;
            // Which shard holds the tile's first element: ONE 64-bit division per tile. A tile spans far fewer elements than a
            // shard, so every other element of it lives in that shard or in the next; the loop below walks on in the rare
            // case of tiny shards.
            const uint64_t tileFlat = d.srcFlatOff + (uint64_t)(d.r0 + rowBase) * colsFull + d.c0 + colBase;
            const uint64_t owner0 = tileFlat / a.shardElems;
            const uint64_t rel0 = tileFlat - owner0 * a.shardElems + (uint64_t)warp * colsFull + lane * 8;
            const uint64_t relStep = (uint64_t)(kThreads / 32) * colsFull;
            const char *ownerBase = shard0 + owner0 * m->symmetricSize;
            uint4 v[kVecPerThread];
#pragma unroll
            for (int i = 0; i < kVecPerThread; i++) {
                const uint32_t r = rowBase + warp + i * (kThreads / 32);
                v[i] = make_uint4(0u, 0u, 0u, 0u);
                if (colOk && r < nrows) {
                    uint64_t within = rel0 + (uint64_t)i * relStep;
                    const char *base = ownerBase;
                    while (within >= a.shardElems) {
                        within -= a.shardElems;
                        base += m->symmetricSize;
                    }
                    v[i] = mf_ld16_coherent(base + within * 2);
                }
            }
            if (d.quant) {
                float amax = 0.f;
#pragma unroll
                for (int i = 0; i < kVecPerThread; i++) {
                    const __nv_bfloat162 *h = reinterpret_cast<const __nv_bfloat162 *>(&v[i]);
#pragma unroll
                    for (int q = 0; q < 4; q++) {
                        float2 f = __bfloat1622float2(h[q]);
                        amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
                    }
                }
                // Lanes 0-15 of every warp hold columns of the tile's left quantisation block, lanes 16-31 of the right one.
#pragma unroll
                for (int o = 8; o > 0; o >>= 1) {
                    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
                }
                const int half = lane >> 4;
                if ((lane & 15) == 0) {
                    warpMax[half][warp] = amax;
                }
                __syncthreads();
                float tmax = 0.f;
#pragma unroll
                for (int w = 0; w < kThreads / 32; w++) {
                    tmax = fmaxf(tmax, warpMax[half][w]);
                }
                __syncthreads();  // warpMax is rewritten by the next tile
                const float sc = fmaxf(tmax, 1e-10f) * (1.f / 448.f);
                const float inv = 1.f / sc;
                unsigned char *dst = reinterpret_cast<unsigned char *>(a.dst) + d.dstOff + c;
#pragma unroll
                for (int i = 0; i < kVecPerThread; i++) {
                    const uint32_t r = rowBase + warp + i * (kThreads / 32);
                    if (colOk && r < nrows) {
                        const __nv_bfloat162 *h = reinterpret_cast<const __nv_bfloat162 *>(&v[i]);
                        uint2 pk;
                        unsigned short *ps = reinterpret_cast<unsigned short *>(&pk);
#pragma unroll
                        for (int q = 0; q < 4; q++) {
                            float2 f = __bfloat1622float2(h[q]);
                            ps[q] = __nv_cvt_float2_to_fp8x2(make_float2(f.x * inv, f.y * inv), __NV_SATFINITE, __NV_E4M3);
                        }
                        *reinterpret_cast<uint2 *>(dst + (size_t)r * ncols) = pk;
                    }
                }
                if ((lane & 15) == 0 && warp == 0 && colBase + half * kTile < ncols) {
                    a.dstScale[d.scaleOff + (size_t)tr * (ncols / kTile) + tc * 2 + half] = sc;
                }
            } else {
                char *dst = reinterpret_cast<char *>(a.dst) + d.dstOff + (size_t)c * 2;
#pragma unroll
                for (int i = 0; i < kVecPerThread; i++) {
                    const uint32_t r = rowBase + warp + i * (kThreads / 32);
                    if (colOk && r < nrows) {
                        mf_st16(dst + (size_t)r * ncols * 2, v[i]);
                    }
                }
            }
        }
    }
    grid.sync();
    if (blockIdx.x == 0 && !dead) {
        int rc = mf_barrier_cta(m, channel, 0, 2 * epoch, timeoutNs);
        if (rc != MF_DEV_OK && threadIdx.x == 0 && a.status != nullptr) {
            atomicCAS(a.status, 0, rc);
        }
    }
}

}  // namespace

extern "C" int mf_k_reshard(const mf_reshard_args_t *argsDev, int nEmulatedRanks, int rankCount, uint32_t channel, uint64_t epoch, uint64_t timeoutNs,
                            int ctas, mf_stream_t stream)
{
    if (argsDev == nullptr || nEmulatedRanks < 1 || rankCount < 1 || rankCount > (int)MF_SIGNAL_MAX_RANKS || channel >= MF_SIGNAL_CHANNELS || epoch == 0) {
        return MF_K_INVALID;
    }
    if (timeoutNs == 0) {
        timeoutNs = 2000000000ull;
    }
    int perSm = 0, dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&perSm, mf_reshard_kernel, kThreads, 0) != cudaSuccess || perSm * sms <= 0) {
        (void)cudaGetLastError();
        return MF_K_LAUNCH_FAILED;
    }
    int grid = perSm * sms / nEmulatedRanks;
    if (ctas > 0 && ctas < grid) {
        grid = ctas;
    }
    if (grid < 1) {
        return MF_K_TOO_LARGE;
    }
    void *kargs[] = {(void *)&argsDev, (void *)&channel, (void *)&epoch, (void *)&timeoutNs};
    dim3 g((unsigned)grid, (unsigned)nEmulatedRanks, 1), b(kThreads, 1, 1);
    cudaError_t e = cudaLaunchCooperativeKernel((const void *)mf_reshard_kernel, g, b, kargs, 0, (cudaStream_t)stream);
    if (e != cudaSuccess) {
        (void)cudaGetLastError();
        return MF_K_LAUNCH_FAILED;
    }
    return MF_K_OK;
}
