// MoE expert-parallel dispatch and combine over the symmetric heap, each as ONE kernel that computes and communicates.
//
// dispatch  (a) histogram of this rank's (token, k) pairs per global expert, pushed to every rank; (b) after a cross-rank
//           barrier every rank knows the full count matrix and derives, without any further message, the row of the
//           destination rank's receive buffer where each of its pairs lands (experts contiguous, starts aligned to the
//           128-row GEMM tile, sources in rank order); (c) each token is quantised ONCE to e4m3 with 1x128 scales in
//           shared memory and its bytes, scales and routing record are stored straight into the receive buffers of the
//           owners of its top-k experts over NVLink; (d) a closing barrier tells the owners that everything has landed.
//           The owner-side tables (expert_offset / expert_count) that the grouped GEMM consumes are written on the way.
// combine   each expert owner pushes its output rows back to the source rank's landing zone [token][k][hidden]; after a
//           barrier the source reduces over k in fp32 with the renormalised routing weights (fixed k order: deterministic)
//           and writes bf16.
// The reference library names MoE dispatch/combine only as a use case of its symmetric heap (README.md:53 of the reference);
// the flag/barrier discipline follows its sample kernel (example/shm/AllReduce/shm_all_reduce.cpp:69-112) with bounded waits.
// Like the all-reduce, both kernels take an array of per-rank argument blocks so that tests can run all ranks of a fake
// heap as gridDim.y slices of one cooperative launch on a single GPU.
#include <cooperative_groups.h>
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

#include "mf/device/mf_shm_device.cuh"
#include "mf_kernels.h"

namespace cg = cooperative_groups;

namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kMaxExperts = 1024;

__device__ __forceinline__ void FailD(int *status, int code)
{
    if (threadIdx.x == 0 && status != nullptr) {
        atomicCAS(status, 0, code);
    }
}

__device__ __forceinline__ int ReadAbort(int *status, int *smemFlag)
{
    if (threadIdx.x == 0) {
        *smemFlag = status != nullptr ? *(volatile int *)status : 0;
    }
    __syncthreads();
    int v = *smemFlag;
    __syncthreads();
    return v;
}

__global__ void __launch_bounds__(kThreads, 1)
mf_moe_dispatch_kernel(const mf_moe_dispatch_args_t *__restrict__ args, int H, int K, int E, uint32_t channel, uint64_t epoch, uint64_t timeoutNs)
{
    cg::grid_group grid = cg::this_grid();
    const mf_moe_dispatch_args_t a = args[blockIdx.y];
    const MfDeviceMeta *m = reinterpret_cast<const MfDeviceMeta *>(a.meta);
    const int R = (int)m->rankCount, me = (int)m->rankId, EL = E / R;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nblk = H / 128;
    extern __shared__ unsigned char smem[];
    int *sendBase = reinterpret_cast<int *>(smem);                              // [E]
    int *totals = sendBase + kMaxExperts;                                       // [E] pairs per expert over all sources
    int *starts = totals + kMaxExperts;                                         // [E] first row of the expert on its owner
    unsigned char *stage = smem + (size_t)3 * kMaxExperts * sizeof(int);        // per warp: H bytes fp8 + nblk floats
    const size_t stagePerWarp = (size_t)H + (size_t)nblk * 4;
    __shared__ int abortFlag;

    // ---- (a) histogram of my pairs per global expert
    const int pairs = a.T * K;
    for (int i = blockIdx.x * kThreads + threadIdx.x; i < pairs; i += gridDim.x * kThreads) {
        const int e = a.topkIdx[i];
        if (e >= 0 && e < E) {
            atomicAdd(&a.localCnt[e], 1);
        }
    }
    __threadfence();
    grid.sync();
    if (blockIdx.x == 0) {
        for (int i = threadIdx.x; i < E * R; i += kThreads) {
            const int r = i / E, e = i % E;
            int *peerCnt = mf_shm_peer(m, a.cnt, (uint32_t)r);
            peerCnt[me * E + e] = ((volatile int *)a.localCnt)[e];
        }
        // Nobody sends before every rank is inside this call (its receive buffers are free) and has published its counts.
        int rc = mf_barrier_cta(m, channel, 0, 2 * epoch - 1, timeoutNs);
        if (rc != MF_DEV_OK) {
            FailD(a.status, rc);
        }
    }
    grid.sync();
    const bool dead = ReadAbort(a.status, &abortFlag) != 0;

    if (!dead) {
        // ---- (b) where my pairs land: sendBase[e] = start of expert e on its owner + pairs of lower ranks for e.
        // Column sums of the count matrix first (one expert per thread, R loads each), then short prefix walks in shared memory.
        for (int e = threadIdx.x; e < E; e += kThreads) {
            int tot = 0, before = 0;
            for (int s = 0; s < R; s++) {
                const int c = ((volatile int *)a.cnt)[s * E + e];
                tot += c;
                before += s < me ? c : 0;
            }
            totals[e] = tot;
            sendBase[e] = before;
        }
        __syncthreads();
        for (int e = threadIdx.x; e < E; e += kThreads) {
            int start = 0;
            for (int e2 = (e / EL) * EL; e2 < e; e2++) {
                start += (totals[e2] + 127) & ~127;
            }
            starts[e] = start;
        }
        __syncthreads();
        for (int e = threadIdx.x; e < E; e += kThreads) {
            sendBase[e] += starts[e];
        }
        if (blockIdx.x == 0) {
            for (int el = threadIdx.x; el < EL; el += kThreads) {
                a.expertOffset[el] = starts[me * EL + el];
                a.expertCount[el] = totals[me * EL + el];
            }
            if (threadIdx.x == 0) {
                const int last = me * EL + EL - 1;
                const int off = starts[last] + ((totals[last] + 127) & ~127);
                a.expertOffset[EL] = off;
                if (off > a.cap) {
                    FailD(a.status, MF_DEV_ERR_BOUNDS);
                }
            }
        }
        __syncthreads();

        // ---- (c) quantise each token once, store it to the owners of its experts
        unsigned char *myStage = stage + (size_t)warp * stagePerWarp;
        float *myScale = reinterpret_cast<float *>(myStage + H);
        const int warpsTotal = gridDim.x * kWarps;
        for (int t = blockIdx.x * kWarps + warp; t < a.T; t += warpsTotal) {
            const __nv_bfloat16 *row = reinterpret_cast<const __nv_bfloat16 *>(a.x) + (size_t)t * H;
            for (int b0 = 0; b0 < nblk; b0 += 2) {
                // Lanes 0-15 own block b0, lanes 16-31 block b0+1; with an odd block count the upper half idles through the
                // same instructions (no divergent shuffles).
                const int blk = b0 + (lane >> 4);
                const bool active = blk < nblk;
                const int off = (active ? blk : b0) * 128 + (lane & 15) * 8;
                uint4 raw = make_uint4(0u, 0u, 0u, 0u);
                if (active) {
                    raw = *reinterpret_cast<const uint4 *>(row + off);
                }
                const __nv_bfloat162 *h = reinterpret_cast<const __nv_bfloat162 *>(&raw);
                float f[8];
                float amax = 0.f;
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    float2 v = __bfloat1622float2(h[i]);
                    f[2 * i] = v.x;
                    f[2 * i + 1] = v.y;
                    amax = fmaxf(amax, fmaxf(fabsf(v.x), fabsf(v.y)));
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
                    *reinterpret_cast<uint2 *>(myStage + off) = packed;
                    if ((lane & 15) == 0) {
                        myScale[blk] = sc;
                    }
                }
            }
            __syncwarp();
            for (int k = 0; k < K; k++) {
                const int e = a.topkIdx[t * K + k];
                if (e < 0 || e >= E) {
                    continue;
                }
                int slot = 0;
                if (lane == 0) {
                    slot = sendBase[e] + atomicAdd(&a.cursor[e], 1);
                    if (a.sendSlot != nullptr) {
                        a.sendSlot[t * K + k] = slot;
                    }
                }
                slot = __shfl_sync(0xffffffffu, slot, 0);
                if (slot >= a.cap) {
                    if (lane == 0 && a.status != nullptr) {
                        atomicCAS(a.status, 0, MF_DEV_ERR_BOUNDS);
                    }
                    continue;
                }
                const uint32_t d = (uint32_t)(e / EL);
                unsigned char *dx = reinterpret_cast<unsigned char *>(mf_shm_peer(m, a.recvX, d)) + (size_t)slot * H;
                float *ds = mf_shm_peer(m, a.recvScale, d) + (size_t)slot * nblk;
                for (int v = lane; v < H / 16; v += 32) {
                    mf_st16(dx + (size_t)v * 16, *reinterpret_cast<const uint4 *>(myStage + (size_t)v * 16));
                }
                for (int v = lane; v < nblk; v += 32) {
                    ds[v] = myScale[v];
                }
                if (lane == 0) {
                    int4 meta = make_int4(me, t, k, __float_as_int(a.topkW[t * K + k]));
                    mf_shm_peer(m, a.recvMeta, d)[slot] = meta;
                }
            }
            __syncwarp();
        }
    }
    // ---- (d) everything I sent is visible before my arrival is; when all have arrived, all receive buffers are complete
    __threadfence_system();
    grid.sync();
    if (blockIdx.x == 0) {
        if (!dead) {
            int rc = mf_barrier_cta(m, channel, 0, 2 * epoch, timeoutNs);
            if (rc != MF_DEV_OK) {
                FailD(a.status, rc);
            }
        }
        // leave the scratch counters clean for the next call
        for (int e = threadIdx.x; e < E; e += kThreads) {
            a.localCnt[e] = 0;
            a.cursor[e] = 0;
        }
    }
}

__global__ void __launch_bounds__(kThreads, 1)
mf_moe_combine_kernel(const mf_moe_combine_args_t *__restrict__ args, int H, int K, int EL, uint32_t channel, uint64_t epoch, uint64_t timeoutNs)
{
    cg::grid_group grid = cg::this_grid();
    const mf_moe_combine_args_t a = args[blockIdx.y];
    const MfDeviceMeta *m = reinterpret_cast<const MfDeviceMeta *>(a.meta);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int warpsTotal = gridDim.x * kWarps;
    __shared__ int offs[kMaxExperts + 1];
    __shared__ int cnts[kMaxExperts];
    __shared__ int abortFlag;
    for (int i = threadIdx.x; i <= EL; i += kThreads) {
        offs[i] = a.expertOffset[i];
        if (i < EL) {
            cnts[i] = a.expertCount[i];
        }
    }
    __syncthreads();
    const int rows = offs[EL];
    const int vecs = H / 8;

    // ---- push: each valid output row goes to its source rank's landing zone [token][k][:]
    for (int r = blockIdx.x * kWarps + warp; r < rows; r += warpsTotal) {
        int el = 0;
        while (el + 1 < EL && offs[el + 1] <= r) {
            el++;
        }
        if (r - offs[el] >= cnts[el]) {
            continue;  // padding row of the tile grid
        }
        const int4 meta = a.recvMeta[r];
        const uint32_t src = (uint32_t)meta.x;
        if (src >= m->rankCount) {
            continue;
        }
        const char *y = reinterpret_cast<const char *>(a.y) + (size_t)r * H * 2;
        char *dst = reinterpret_cast<char *>(mf_shm_peer(m, a.retY, src)) + ((size_t)meta.y * K + meta.z) * H * 2;
        for (int v = lane; v < vecs; v += 32) {
            mf_st16(dst + (size_t)v * 16, mf_ld16(y + (size_t)v * 16));
        }
    }
    __threadfence_system();
    grid.sync();
    if (blockIdx.x == 0) {
        int rc = mf_barrier_cta(m, channel, 0, epoch, timeoutNs);
        if (rc != MF_DEV_OK) {
            FailD(a.status, rc);
        }
    }
    grid.sync();
    if (ReadAbort(a.status, &abortFlag) != 0) {
        return;
    }
    // ---- reduce over k with the routing weights (fp32, fixed order)
    for (int t = blockIdx.x * kWarps + warp; t < a.T; t += warpsTotal) {
        const char *base = reinterpret_cast<const char *>(a.retY) + (size_t)t * K * H * 2;
        char *o = reinterpret_cast<char *>(a.out) + (size_t)t * H * 2;
        for (int v = lane; v < vecs; v += 32) {
            float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            for (int k = 0; k < K; k++) {
                const float w = a.topkW[t * K + k];
                const uint4 raw = mf_ld16_coherent(base + (size_t)k * H * 2 + (size_t)v * 16);
                const __nv_bfloat162 *h = reinterpret_cast<const __nv_bfloat162 *>(&raw);
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    float2 f = __bfloat1622float2(h[i]);
                    acc[2 * i] = fmaf(w, f.x, acc[2 * i]);
                    acc[2 * i + 1] = fmaf(w, f.y, acc[2 * i + 1]);
                }
            }
            uint4 pk;
            __nv_bfloat162 *hp = reinterpret_cast<__nv_bfloat162 *>(&pk);
#pragma unroll
            for (int i = 0; i < 4; i++) {
                hp[i] = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
            }
            mf_st16(o + (size_t)v * 16, pk);
        }
    }
}

int CoopCap(const void *kernel, size_t smem)
{
    int perSm = 0, dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&perSm, kernel, kThreads, smem) != cudaSuccess) {
        (void)cudaGetLastError();
        return 0;
    }
    return perSm * sms;
}

}  // namespace

extern "C" int mf_k_moe_dispatch(const mf_moe_dispatch_args_t *argsDev, int nEmulatedRanks, int rankCount, int H, int K, int E, uint32_t channel,
                                 uint64_t epoch, uint64_t timeoutNs, int ctas, mf_stream_t stream)
{
    if (argsDev == nullptr || nEmulatedRanks < 1 || rankCount < 1 || rankCount > (int)MF_SIGNAL_MAX_RANKS || H <= 0 || H % 128 != 0 || K < 1 ||
        K > 32 || E < rankCount || E % rankCount != 0 || E > kMaxExperts || channel >= MF_SIGNAL_CHANNELS || epoch == 0) {
        return MF_K_INVALID;
    }
    if (timeoutNs == 0) {
        timeoutNs = 2000000000ull;
    }
    const size_t smem = (size_t)3 * kMaxExperts * sizeof(int) + (size_t)kWarps * ((size_t)H + (size_t)(H / 128) * 4);
    static size_t attrSmem = 0;
    if (smem > attrSmem) {
        if (cudaFuncSetAttribute(mf_moe_dispatch_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
            (void)cudaGetLastError();
            return MF_K_TOO_LARGE;
        }
        attrSmem = smem;
    }
    int cap = CoopCap((const void *)mf_moe_dispatch_kernel, smem);
    if (cap <= 0) {
        return MF_K_LAUNCH_FAILED;
    }
    int grid = cap / nEmulatedRanks;
    if (ctas > 0 && ctas < grid) {
        grid = ctas;
    }
    if (grid < 1) {
        return MF_K_TOO_LARGE;
    }
    void *kargs[] = {(void *)&argsDev, (void *)&H, (void *)&K, (void *)&E, (void *)&channel, (void *)&epoch, (void *)&timeoutNs};
    dim3 g((unsigned)grid, (unsigned)nEmulatedRanks, 1), b(kThreads, 1, 1);
    cudaError_t e = cudaLaunchCooperativeKernel((const void *)mf_moe_dispatch_kernel, g, b, kargs, smem, (cudaStream_t)stream);
    if (e != cudaSuccess) {
        (void)cudaGetLastError();
        return MF_K_LAUNCH_FAILED;
    }
    return MF_K_OK;
}

extern "C" int mf_k_moe_combine(const mf_moe_combine_args_t *argsDev, int nEmulatedRanks, int rankCount, int H, int K, int EL, uint32_t channel,
                                uint64_t epoch, uint64_t timeoutNs, int ctas, mf_stream_t stream)
{
    if (argsDev == nullptr || nEmulatedRanks < 1 || rankCount < 1 || rankCount > (int)MF_SIGNAL_MAX_RANKS || H <= 0 || H % 8 != 0 || K < 1 || K > 32 ||
        EL < 1 || EL > kMaxExperts || channel >= MF_SIGNAL_CHANNELS || epoch == 0) {
        return MF_K_INVALID;
    }
    if (timeoutNs == 0) {
        timeoutNs = 2000000000ull;
    }
    int cap = CoopCap((const void *)mf_moe_combine_kernel, 0);
    if (cap <= 0) {
        return MF_K_LAUNCH_FAILED;
    }
    int grid = cap / nEmulatedRanks;
    if (ctas > 0 && ctas < grid) {
        grid = ctas;
    }
    if (grid < 1) {
        return MF_K_TOO_LARGE;
    }
    void *kargs[] = {(void *)&argsDev, (void *)&H, (void *)&K, (void *)&EL, (void *)&channel, (void *)&epoch, (void *)&timeoutNs};
    dim3 g((unsigned)grid, (unsigned)nEmulatedRanks, 1), b(kThreads, 1, 1);
    cudaError_t e = cudaLaunchCooperativeKernel((const void *)mf_moe_combine_kernel, g, b, kargs, 0, (cudaStream_t)stream);
    if (e != cudaSuccess) {
        (void)cudaGetLastError();
        return MF_K_LAUNCH_FAILED;
    }
    return MF_K_OK;
}
