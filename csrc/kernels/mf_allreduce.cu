// Fused all-reduce + residual add + RMSNorm over the symmetric heap:
//     h   = residual + sum_r x_r            (new residual, bf16)
//     out = h * rsqrt(mean(h^2) + eps) * w  (bf16)
// in ONE kernel that reads peers' x (or reduces it inside NVSwitch) and applies the norm on the same rows. The collective
// contract is the reference's sample all-reduce (sum over ranks, every rank gets the full result, flag barrier before and
// after; example/shm/AllReduce/shm_all_reduce.cpp:45-135) widened from its fixed 16x2048 fp16 shape to [T, H] bf16 with the
// transformer epilogue fused in. Three algorithms, chosen per size:
//   one-shot   every rank pulls all R copies of every row and reduces locally. Latency-optimal for small inputs.
//   two-shot   rank r reduces rows [rT/R, (r+1)T/R) from all peers, adds the residual and pushes the new residual row to
//              every rank; after a cross-rank barrier every rank normalises all rows locally. NVLink carries 2(R-1)/R of
//              the tensor per direction — the all-reduce minimum — and the norm never makes a separate pass over x.
//   nvls       same schedule, but the reduction is a multimem.ld_reduce executed by NVSwitch and the broadcast a
//              multimem.st: each GPU moves ~1x the tensor per direction instead of ~2x.
// Accumulation is fp32 in rank order, so every rank computes bit-identical results. All cross-rank waits are bounded:
// on expiry the kernel stores an error code to *status and every CTA leaves through the normal exit.
// The launcher takes an array of per-rank argument blocks: production passes one; tests that emulate R ranks on a single
// GPU pass R and the kernel runs them as gridDim.y slices of one cooperative launch (separate launches that wait on one
// another are never used).
#include <cooperative_groups.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <mutex>

#include "mf/device/mf_shm_device.cuh"
#include "mf_kernels.h"

namespace cg = cooperative_groups;

namespace {

constexpr int kThreads = 512;
constexpr int kMaxVpt = 4;  // 16-byte vectors per thread per row: H <= 512 * 4 * 8 = 16384

struct Acc8 {
    float v[8];
};

__device__ __forceinline__ void Unpack(const uint4 &u, float *f)
{
    const __nv_bfloat162 *p = reinterpret_cast<const __nv_bfloat162 *>(&u);
#pragma unroll
    for (int i = 0; i < 4; i++) {
        float2 t = __bfloat1622float2(p[i]);
        f[2 * i] = t.x;
        f[2 * i + 1] = t.y;
    }
}

__device__ __forceinline__ uint4 Pack(const float *f)
{
    uint4 u;
    __nv_bfloat162 *p = reinterpret_cast<__nv_bfloat162 *>(&u);
#pragma unroll
    for (int i = 0; i < 4; i++) {
        p[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
    }
    return u;
}

__device__ __forceinline__ float BlockSum(float v)
{
    __shared__ float warpSums[kThreads / 32];
    __shared__ float total;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        v += __shfl_xor_sync(0xffffffffu, v, o);
    }
    if ((threadIdx.x & 31) == 0) {
        warpSums[threadIdx.x >> 5] = v;
    }
    __syncthreads();
    if (threadIdx.x < 32) {
        float s = threadIdx.x < kThreads / 32 ? warpSums[threadIdx.x] : 0.f;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            s += __shfl_xor_sync(0xffffffffu, s, o);
        }
        if (threadIdx.x == 0) {
            total = s;
        }
    }
    __syncthreads();
    float r = total;
    __syncthreads();  // `total` may be rewritten by the next row
    return r;
}

// Sum over ranks of one 16-byte vector at heap-symmetric address `xLocal + byteOff`, fp32, rank order 0..R-1.
__device__ __forceinline__ void ReduceVec(const MfDeviceMeta *m, const char *xLocal, size_t byteOff, float *acc)
{
    const uint32_t R = m->rankCount;
#pragma unroll
    for (int i = 0; i < 8; i++) {
        acc[i] = 0.f;
    }
    const char *rank0 = xLocal - (uint64_t)m->rankId * m->symmetricSize + byteOff;
    for (uint32_t r0 = 0; r0 < R; r0 += 8) {
        uint4 v[8];
        const uint32_t n = min(8u, R - r0);
#pragma unroll
        for (uint32_t j = 0; j < 8; j++) {
            if (j < n) {
                v[j] = mf_ld16_coherent(rank0 + (uint64_t)(r0 + j) * m->symmetricSize);
            }
        }
#pragma unroll
        for (uint32_t j = 0; j < 8; j++) {
            if (j < n) {
                float f[8];
                Unpack(v[j], f);
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    acc[i] += f[i];
                }
            }
        }
    }
}

// Normalises one row held in registers (already rounded to bf16 precision) and stores `out`.
template <int VPT>
__device__ __forceinline__ void NormAndStore(Acc8 (&row)[VPT], int vecsPerRow, const char *weight, char *outRow, int H, float eps)
{
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < VPT; k++) {
        if ((int)threadIdx.x + k * kThreads < vecsPerRow) {
#pragma unroll
            for (int i = 0; i < 8; i++) {
                ss += row[k].v[i] * row[k].v[i];
            }
        }
    }
    ss = BlockSum(ss);
    const float rstd = rsqrtf(ss / (float)H + eps);
#pragma unroll
    for (int k = 0; k < VPT; k++) {
        const int vec = (int)threadIdx.x + k * kThreads;
        if (vec < vecsPerRow) {
            float w[8], o[8];
            Unpack(*reinterpret_cast<const uint4 *>(weight + (size_t)vec * 16), w);
#pragma unroll
            for (int i = 0; i < 8; i++) {
                o[i] = row[k].v[i] * rstd * w[i];
            }
            mf_st16(outRow + (size_t)vec * 16, Pack(o));
        }
    }
}

__device__ __forceinline__ void RoundToBf16(float *f)
{
#pragma unroll
    for (int i = 0; i < 8; i++) {
        f[i] = __bfloat162float(__float2bfloat16_rn(f[i]));
    }
}

__device__ __forceinline__ void Fail(const mf_allreduce_args_t &a, int code)
{
    if (threadIdx.x == 0 && a.status != nullptr) {
        atomicCAS(a.status, 0, code);
    }
}

// Epoch of this call: the kernel argument, or (argument 0) one more than the device-resident count of finished calls. Every CTA
// of the launch reads the same value: the count only moves when the LAST CTA of a launch retires (FinishEpoch).
__device__ __forceinline__ uint64_t ResolveEpoch(const mf_allreduce_args_t &a, uint64_t epochArg)
{
    if (epochArg != 0 || a.epochState == nullptr) {
        return epochArg;
    }
    return *(volatile unsigned long long *)a.epochState + 1;
}

// Called by every CTA on every way out of the kernel (after its last use of the epoch).
__device__ __forceinline__ void FinishEpoch(const mf_allreduce_args_t &a, uint64_t epochArg, uint64_t epoch)
{
    if (epochArg != 0 || a.epochState == nullptr) {
        return;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        const unsigned long long done = atomicAdd(a.epochState + 1, 1ull);
        if (done == (unsigned long long)gridDim.x - 1) {
            a.epochState[1] = 0;
            *(volatile unsigned long long *)a.epochState = epoch;
            __threadfence();
        }
    }
}

// ------------------------------------------------------------------------------------------------ one-shot

template <int VPT, bool TAIL>
__global__ void __launch_bounds__(kThreads, 1)
mf_allreduce_rmsnorm_oneshot_kernel(const mf_allreduce_args_t *__restrict__ args, int T, int H, float eps, uint32_t channel, uint64_t epochArg,
                                    uint64_t timeoutNs)
{
    const mf_allreduce_args_t a = args[blockIdx.y];
    const MfDeviceMeta *m = reinterpret_cast<const MfDeviceMeta *>(a.meta);
    const int vecsPerRow = H / 8;
    const uint64_t epoch = ResolveEpoch(a, epochArg);
    if (mf_check_bounds_enabled(m) && !mf_shm_in_own_window(m, a.x, (uint64_t)T * H * 2)) {
        Fail(a, MF_DEV_ERR_BOUNDS);  // peers would read my x at this offset of their own heaps: it must be heap memory
        FinishEpoch(a, epochArg, epoch);
        return;
    }
    // Peers' x is complete once their CTA of the same index has arrived here.
    int rc = mf_barrier_cta(m, channel, blockIdx.x, 2 * epoch - 1, timeoutNs);
    if (rc != MF_DEV_OK) {
        Fail(a, rc);
        FinishEpoch(a, epochArg, epoch);
        return;
    }
    for (int row = blockIdx.x; row < T; row += gridDim.x) {
        const size_t rowOff = (size_t)row * H * 2;
        Acc8 acc[VPT];
#pragma unroll
        for (int k = 0; k < VPT; k++) {
            const int vec = (int)threadIdx.x + k * kThreads;
            if (vec < vecsPerRow) {
                ReduceVec(m, (const char *)a.x, rowOff + (size_t)vec * 16, acc[k].v);
                if (a.residual != nullptr) {
                    float res[8];
                    Unpack(mf_ld16((const char *)a.residual + rowOff + (size_t)vec * 16), res);
#pragma unroll
                    for (int i = 0; i < 8; i++) {
                        acc[k].v[i] += res[i];
                    }
                }
                RoundToBf16(acc[k].v);
                if (a.residualOut != nullptr) {
                    mf_st16((char *)a.residualOut + rowOff + (size_t)vec * 16, Pack(acc[k].v));
                }
            }
        }
        NormAndStore<VPT>(acc, vecsPerRow, (const char *)a.weight, (char *)a.out + rowOff, H, eps);
    }
    // Nobody may overwrite its x before every rank has finished reading it. Callers that alternate between two x buffers get
    // that guarantee from the opening barrier of their next call and skip this round trip.
    if (TAIL) {
        rc = mf_barrier_cta(m, channel, blockIdx.x, 2 * epoch, timeoutNs);
        if (rc != MF_DEV_OK) {
            Fail(a, rc);
        }
    }
    FinishEpoch(a, epochArg, epoch);
}

// ------------------------------------------------------------------------------------------------ two-shot / NVLS

// RC: compile-time upper bound of the rank count (2, 4 or 8; 0 = any) so that the peer vectors of a trip live in registers.
template <bool NVLS, int VPT, int RC>
__global__ void __launch_bounds__(kThreads, 1)
mf_allreduce_rmsnorm_twoshot_kernel(const mf_allreduce_args_t *__restrict__ args, int T, int H, float eps, uint32_t channel, uint64_t epochArg,
                                    uint64_t timeoutNs)
{
    cg::grid_group grid = cg::this_grid();
    const mf_allreduce_args_t a = args[blockIdx.y];
    const MfDeviceMeta *m = reinterpret_cast<const MfDeviceMeta *>(a.meta);
    const uint32_t R = m->rankCount, me = m->rankId;
    const int vecsPerRow = H / 8;
    const uint64_t epoch = ResolveEpoch(a, epochArg);
    __shared__ int abortFlag;
    if (mf_check_bounds_enabled(m) && !(mf_shm_in_own_window(m, a.x, (uint64_t)T * H * 2) && mf_shm_in_own_window(m, a.residualOut, (uint64_t)T * H * 2))) {
        Fail(a, MF_DEV_ERR_BOUNDS);  // every CTA of every rank decides alike from the same arguments: nobody waits for anybody
        FinishEpoch(a, epochArg, epoch);
        return;
    }

    // Phase 0: every rank's x is ready. One CTA per rank shakes hands, the grid barrier spreads the news.
    if (blockIdx.x == 0) {
        int rc = mf_barrier_cta(m, channel, 0, 2 * epoch - 1, timeoutNs);
        if (rc != MF_DEV_OK) {
            Fail(a, rc);
        }
    }
    grid.sync();
    if (threadIdx.x == 0) {
        abortFlag = a.status != nullptr ? *(volatile int *)a.status : 0;
    }
    __syncthreads();
    const bool dead = abortFlag != 0;  // after a timeout keep walking through the grid barriers, touch no peer memory

    // Phase 1: reduce my block of rows, add the residual, push the new residual row to every rank.
    const int rowLo = (int)(((long long)T * me) / R), rowHi = (int)(((long long)T * (me + 1)) / R);
    if (!dead) {
        const int64_t heapOffX = (const char *)a.x - (const char *)mf_shm_ptr(m, me, 0);
        const int64_t heapOffRes = (char *)a.residualOut - (char *)mf_shm_ptr(m, me, 0);
        // Phase 1 needs no row structure (the norm happens in phase 2), so it is a flat sweep over the 16-byte vectors of my
        // row block with up to 16 peer vectors in flight per thread: U consecutive tiles of blockDim vectors per trip.
        const char *rank0x = (const char *)a.x - (uint64_t)me * m->symmetricSize;
        const size_t firstVec = (size_t)rowLo * vecsPerRow, nVec = (size_t)(rowHi - rowLo) * vecsPerRow;
        constexpr int U = NVLS ? 2 : (RC == 2 ? 8 : (RC == 4 ? 4 : (RC == 8 ? 2 : 1)));  // in-switch reductions: two in flight measured best
        constexpr int RCC = RC == 0 ? 1 : RC;
        const size_t trip = (size_t)U * kThreads;
        for (size_t base = (size_t)blockIdx.x * trip; base < nVec; base += (size_t)gridDim.x * trip) {
            uint4 in[U][RCC];
            uint4 resv[U];
#pragma unroll
            for (int u = 0; u < U; u++) {
                const size_t i = base + (size_t)u * kThreads + threadIdx.x;
                if (i < nVec) {
                    const size_t off = (firstVec + i) * 16;
                    if (NVLS) {
                        in[u][0] = mf_multimem_ld_reduce_add_bf16x8((const char *)m->multicastBase + heapOffX + off);
                    } else if (RC != 0) {
#pragma unroll
                        for (uint32_t j = 0; j < (uint32_t)RCC; j++) {
                            if (j < R) {
                                in[u][j] = mf_ld16_coherent(rank0x + (uint64_t)j * m->symmetricSize + off);
                            }
                        }
                    }
                    if (a.residual != nullptr) {
                        resv[u] = mf_ld16((const char *)a.residual + off);
                    }
                }
            }
#pragma unroll
            for (int u = 0; u < U; u++) {
                const size_t i = base + (size_t)u * kThreads + threadIdx.x;
                if (i < nVec) {
                    const size_t off = (firstVec + i) * 16;
                    float acc[8];
                    if (NVLS) {
                        Unpack(in[u][0], acc);
                    } else if (RC != 0) {
#pragma unroll
                        for (int q = 0; q < 8; q++) {
                            acc[q] = 0.f;
                        }
#pragma unroll
                        for (uint32_t j = 0; j < (uint32_t)RCC; j++) {
                            if (j < R) {
                                float f[8];
                                Unpack(in[u][j], f);
#pragma unroll
                                for (int q = 0; q < 8; q++) {
                                    acc[q] += f[q];
                                }
                            }
                        }
                    } else {
                        ReduceVec(m, (const char *)a.x, off, acc);
                    }
                    if (a.residual != nullptr) {
                        float res[8];
                        Unpack(resv[u], res);
#pragma unroll
                        for (int q = 0; q < 8; q++) {
                            acc[q] += res[q];
                        }
                    }
                    const uint4 packed = Pack(acc);
                    if (NVLS) {
                        mf_multimem_st16((char *)m->multicastBase + heapOffRes + off, packed);
                    } else {
                        for (uint32_t r = 0; r < R; r++) {
                            mf_st16((char *)mf_shm_ptr(m, (me + r) % R, (uint64_t)heapOffRes + off), packed);
                        }
                    }
                }
            }
        }
    }
    __threadfence_system();
    grid.sync();
    // Phase 1.5: all ranks have pushed. Again one CTA per rank, then the grid barrier.
    if (blockIdx.x == 0 && !dead) {
        int rc = mf_barrier_cta(m, channel, 0, 2 * epoch, timeoutNs);
        if (rc != MF_DEV_OK) {
            Fail(a, rc);
        }
    }
    grid.sync();
    if (threadIdx.x == 0) {
        abortFlag = a.status != nullptr ? *(volatile int *)a.status : 0;
    }
    __syncthreads();
    if (abortFlag != 0) {
        FinishEpoch(a, epochArg, epoch);
        return;
    }
    // Phase 2: normalise every row from the (now complete) local copy of the new residual.
    for (int row = blockIdx.x; row < T; row += gridDim.x) {
        const size_t rowOff = (size_t)row * H * 2;
        Acc8 acc[VPT];
#pragma unroll
        for (int k = 0; k < VPT; k++) {
            const int vec = (int)threadIdx.x + k * kThreads;
            if (vec < vecsPerRow) {
                Unpack(mf_ld16_coherent((const char *)a.residualOut + rowOff + (size_t)vec * 16), acc[k].v);
            }
        }
        NormAndStore<VPT>(acc, vecsPerRow, (const char *)a.weight, (char *)a.out + rowOff, H, eps);
    }
    FinishEpoch(a, epochArg, epoch);
}

template <int VPT>
const void *PickKernel(int algo, int rankCount)
{
    if (algo == MF_AR_ONESHOT) {
        return (const void *)mf_allreduce_rmsnorm_oneshot_kernel<VPT, true>;
    }
    if (algo == MF_AR_ONESHOT_NOTAIL) {
        return (const void *)mf_allreduce_rmsnorm_oneshot_kernel<VPT, false>;
    }
    if (algo == MF_AR_NVLS) {
        return (const void *)mf_allreduce_rmsnorm_twoshot_kernel<true, VPT, 0>;
    }
    if (rankCount <= 2) {
        return (const void *)mf_allreduce_rmsnorm_twoshot_kernel<false, VPT, 2>;
    }
    if (rankCount <= 4) {
        return (const void *)mf_allreduce_rmsnorm_twoshot_kernel<false, VPT, 4>;
    }
    if (rankCount <= 8) {
        return (const void *)mf_allreduce_rmsnorm_twoshot_kernel<false, VPT, 8>;
    }
    return (const void *)mf_allreduce_rmsnorm_twoshot_kernel<false, VPT, 0>;
}

int CoopCapacityQuery(const void *kernel)
{
    int perSm = 0, dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&perSm, kernel, kThreads, 0) != cudaSuccess) {
        (void)cudaGetLastError();
        return 0;
    }
    return perSm * sms;
}

// Resident-CTA capacity of a kernel on the current device. The occupancy query costs microseconds, which is real money on a
// 10 us call path: the answer is remembered per (device, kernel).
int CoopCapacity(const void *kernel)
{
    struct Entry {
        const void *kernel;
        int dev;
        int capacity;
    };
    static Entry cache[64];
    static int used = 0;
    static std::mutex mu;
    int curDev = 0;
    if (cudaGetDevice(&curDev) != cudaSuccess) {
        (void)cudaGetLastError();
        return 0;
    }
    {
        std::lock_guard<std::mutex> g(mu);
        for (int i = 0; i < used; i++) {
            if (cache[i].kernel == kernel && cache[i].dev == curDev) {
                return cache[i].capacity;
            }
        }
    }
    int cap = CoopCapacityQuery(kernel);
    if (cap > 0) {
        std::lock_guard<std::mutex> g(mu);
        if (used < 64) {
            cache[used++] = Entry{kernel, curDev, cap};
        }
    }
    return cap;
}

}  // namespace

extern "C" int mf_k_allreduce_rmsnorm(const mf_allreduce_args_t *argsDev, int nEmulatedRanks, int rankCount, int T, int H, float eps, int algo,
                                      uint32_t channel, uint64_t epoch, uint64_t timeoutNs, int ctas, mf_stream_t stream)
{
    if (argsDev == nullptr || nEmulatedRanks < 1 || rankCount < 1 || rankCount > (int)MF_SIGNAL_MAX_RANKS || T <= 0 || H <= 0 || H % 8 != 0 ||
        H > kThreads * kMaxVpt * 8 || channel >= MF_SIGNAL_CHANNELS) {
        return MF_K_INVALID;  // epoch 0 = device-resident epoch (args->epochState), see the header
    }
    if (timeoutNs == 0) {
        timeoutNs = 2000000000ull;
    }
    const size_t bytes = (size_t)T * H * 2;
    if (algo == MF_AR_AUTO) {
        algo = bytes <= (512u << 10) ? MF_AR_ONESHOT : MF_AR_TWOSHOT;
    }
    void *kargs[] = {(void *)&argsDev, (void *)&T, (void *)&H, (void *)&eps, (void *)&channel, (void *)&epoch, (void *)&timeoutNs};
    // Vectors per thread per row are a compile-time constant so that a row lives in registers.
    const int vecsPerRow = H / 8;
    const void *kernel = vecsPerRow <= kThreads       ? PickKernel<1>(algo, rankCount)
                         : vecsPerRow <= 2 * kThreads ? PickKernel<2>(algo, rankCount)
                                                      : PickKernel<4>(algo, rankCount);
    int capacity = CoopCapacity(kernel);
    if (capacity <= 0) {
        return MF_K_LAUNCH_FAILED;
    }
    int perRank = capacity / nEmulatedRanks;
    int grid;
    const bool oneshot = algo == MF_AR_ONESHOT || algo == MF_AR_ONESHOT_NOTAIL;
    if (oneshot) {
        grid = T < (int)MF_SIGNAL_SLOTS ? T : (int)MF_SIGNAL_SLOTS;  // one signal slot per CTA
    } else {
        int rowsMine = (T + rankCount - 1) / rankCount;
        grid = T < perRank ? T : perRank;
        (void)rowsMine;
    }
    if (ctas > 0 && ctas < grid) {
        grid = ctas;
    }
    if (grid > perRank) {
        grid = perRank;
    }
    if (grid < 1) {
        return MF_K_TOO_LARGE;
    }
    dim3 g((unsigned)grid, (unsigned)nEmulatedRanks, 1), b(kThreads, 1, 1);
    // Cooperative launch: all CTAs (and, when emulating, all ranks) are co-resident, so the waits inside can complete. The
    // one-shot kernel of a real rank needs neither a grid barrier nor co-residency on this GPU (each of its at most 64 CTAs only
    // waits for the CTA of the same index on the OTHER GPUs) and takes the cheaper ordinary launch.
    cudaError_t e = (oneshot && nEmulatedRanks == 1) ? cudaLaunchKernel(kernel, g, b, kargs, 0, (cudaStream_t)stream)
                                                     : cudaLaunchCooperativeKernel(kernel, g, b, kargs, 0, (cudaStream_t)stream);
    if (e != cudaSuccess) {
        (void)cudaGetLastError();
        return MF_K_LAUNCH_FAILED;
    }
    return MF_K_OK;
}
