// MoE expert-parallel dispatch and combine over the symmetric heap, each as ONE kernel that computes and communicates.
//
// dispatch  (a) histogram of this rank's (token, k) pairs per global expert, pushed to every rank; (b) after a cross-rank
//           barrier every rank knows the full count matrix and derives, without any further message, the row of the
//           destination rank's receive buffer where each of its pairs lands (experts contiguous, starts aligned to the
//           128-row GEMM tile, sources in rank order); (c) each token is quantised ONCE to e4m3 with 1x128 power-of-two
//           scales (UE8M0 exponent bytes, the format the block-scaled tensor-core GEMM consumes) in shared memory and its
//           bytes, scale words and routing record are stored straight into the receive buffers of the owners of its top-k
//           experts over NVLink; (d) a closing barrier tells the owners that everything has landed.
//           The owner-side tables (expert_offset / expert_count) that the grouped GEMM consumes are written on the way,
//           clamped to the capacity of the receive buffer: on overflow the call reports MF_DEV_ERR_BOUNDS and what was
//           published never points past the buffer.
//           A token whose top-k holds several experts of the same owner tells that owner, in the record of the first of
//           them (the "leader"), where its sibling rows are.
//           Arrival mode (args.arrive set): instead of (d) every row that has landed is counted, with release semantics, in a
//           counter of its 128-row tile on the owner; the kernel ends without a closing barrier and the grouped GEMM that
//           follows starts each tile when the counter of that tile is complete (mf_k_moe_grouped_gemm_mx_gated), so an owner
//           computes on what has arrived while slower senders are still pushing. Every pair carries its payload in this mode.
// combine   each expert owner reduces the sibling rows of a token with their routing weights (fp32) and pushes ONE row
//           per (token, owner) back to the source rank's landing zone [token][k of the leader][hidden]; after a barrier the
//           source adds the partial sums of the owners in fixed k order (fp32, deterministic) and writes bf16. A top-8
//           token over 8 ranks reaches 5.25 distinct owners on average, so a third of the return traffic never leaves
//           the owner.
// The reference library names MoE dispatch/combine only as a use case of its symmetric heap (README.md:53 of the reference);
// the flag/barrier discipline follows its sample kernel (example/shm/AllReduce/shm_all_reduce.cpp:69-112) with bounded waits.
// Like the all-reduce, both kernels take an array of per-rank argument blocks so that tests can run all ranks of a fake
// heap as gridDim.y slices of one cooperative launch on a single GPU.
#include <cooperative_groups.h>
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

#include <mutex>

#include "mf/device/mf_shm_device.cuh"
#include "mf_kernels.h"

namespace cg = cooperative_groups;

namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kMaxExperts = 1024;
// A token routed to several experts of one owner crosses the link once and is replicated by the owner when the call moves at
// least this many (token, expert) pairs per rank on average; below it the scan of the receive buffer that the replication
// needs costs more than the link time it saves (measured on two GPUs, top-8 of 64 experts: 128 tokens per rank 45 us without
// and 109 us with it, 4096 tokens per rank 233 us without and 190 us with it).
constexpr int kDedupMinPairsPerRank = 8192;

__device__ __forceinline__ void FailD(int *status, int code)
{
    if (threadIdx.x == 0 && status != nullptr) {
        atomicCAS(status, 0, code);
    }
}

// UE8M0 byte (biased exponent) of the smallest power of two >= t, clamped to [1, 253] so that its reciprocal is a normal float.
__device__ __forceinline__ uint32_t Ue8m0Ceil(float t)
{
    const uint32_t bits = __float_as_uint(t);
    const uint32_t e = ((bits >> 23) & 0xffu) + ((bits & 0x7fffffu) != 0u ? 1u : 0u);
    return e < 1u ? 1u : (e > 253u ? 253u : e);
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

// Epoch of this call: the kernel argument, or (argument 0) one more than the device-resident count of finished calls. Every CTA
// of the launch reads the same value: the count only moves when the LAST CTA of a launch retires (FinishEpochD).
template <typename Args>
__device__ __forceinline__ uint64_t ResolveEpochD(const Args &a, uint64_t epochArg)
{
    if (epochArg != 0 || a.epochState == nullptr) {
        return epochArg;
    }
    return *(volatile unsigned long long *)a.epochState + 1;
}

// Called by every thread of every CTA on every way out of the kernel (after its last use of the epoch).
template <typename Args>
__device__ __forceinline__ void FinishEpochD(const Args &a, uint64_t epochArg, uint64_t epoch)
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

// Meta words are written by other GPUs during this kernel: read them past the non-coherent path.
__device__ __forceinline__ int4 mf_ld_meta(const int4 *p)
{
    const uint4 u = mf_ld16_coherent(p);
    return make_int4((int)u.x, (int)u.y, (int)u.z, (int)u.w);
}

// Two CTAs per SM (71 KB of shared memory and at most 128 registers each): a warp works on one token at a time through chains
// of dependent loads, shuffles and stores, so the kernel lives on the number of warps in flight, not on any one unit.
__global__ void __launch_bounds__(kThreads, 2)
mf_moe_dispatch_kernel(const mf_moe_dispatch_args_t *__restrict__ args, int H, int K, int E, uint32_t channel, uint64_t epochArg, uint64_t timeoutNs)
{
    cg::grid_group grid = cg::this_grid();
    const mf_moe_dispatch_args_t a = args[blockIdx.y];
    const uint64_t epoch = ResolveEpochD(a, epochArg);
    if (epoch == 0) {
        FailD(a.status, MF_DEV_ERR_BOUNDS);  // neither an epoch argument nor a device-resident epoch
        return;
    }
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
    __shared__ int grandTotal;
    if (mf_check_bounds_enabled(m) &&
        !(mf_shm_in_own_window(m, a.cnt, (uint64_t)(a.arrive != nullptr ? 2 : 1) * R * E * 4) &&
          (a.arrive == nullptr || mf_shm_in_own_window(m, a.arrive, (uint64_t)(a.cap / 128) * 4)) && mf_shm_in_own_window(m, a.recvX, (uint64_t)a.cap * H) &&
          mf_shm_in_own_window(m, a.recvSf, (uint64_t)a.cap * nblk * 4) && mf_shm_in_own_window(m, a.recvMeta, (uint64_t)a.cap * 16) &&
          mf_shm_in_own_window(m, a.recvSib, (uint64_t)a.cap * MF_MOE_MAX_SIBLINGS * 8))) {
        FailD(a.status, MF_DEV_ERR_BOUNDS);  // the receive buffers are addressed by offset on every owner: they must be heap memory
        FinishEpochD(a, epochArg, epoch);
        return;
    }

    // ---- (a) histogram of my pairs per global expert
    const bool arrival = a.arrive != nullptr;
    const int *myCnt = a.cnt + (arrival ? (size_t)(epoch & 1) * R * E : 0);
    if (arrival) {
        // My tile counters start from zero before anybody is told (by the barrier below) that it may send.
        for (int i = blockIdx.x * kThreads + threadIdx.x; i < a.cap / 128; i += gridDim.x * kThreads) {
            a.arrive[i] = 0;
        }
    }
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
            int *peerCnt = mf_shm_peer(m, const_cast<int *>(myCnt), (uint32_t)r);
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
    bool dedup = false;

    if (!dead) {
        // ---- (b) where my pairs land: sendBase[e] = start of expert e on its owner + pairs of lower ranks for e.
        // Column sums of the count matrix first (one expert per thread, R loads each), then short prefix walks in shared memory.
        for (int e = threadIdx.x; e < E; e += kThreads) {
            int tot = 0, before = 0;
            for (int s = 0; s < R; s++) {
                const int c = ((volatile const int *)myCnt)[s * E + e];
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
        if (warp == 0) {
            // Every rank holds the same count matrix, so every CTA of every rank takes the same decision.
            int sum = 0;
            for (int e = lane; e < E; e += 32) {
                sum += totals[e];
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                sum += __shfl_xor_sync(0xffffffffu, sum, o);
            }
            if (lane == 0) {
                grandTotal = sum;
            }
        }
        __syncthreads();
        dedup = !arrival && (long long)grandTotal >= (long long)R * (a.dedupMinPairs > 0 ? a.dedupMinPairs : kDedupMinPairsPerRank);
        if (blockIdx.x == 0) {
            // What the GEMM and combine consume never points past the receive buffer: an expert that starts beyond the
            // capacity is published empty, one that straddles it is cut. The senders skip the same rows.
            for (int el = threadIdx.x; el < EL; el += kThreads) {
                const int off = min(starts[me * EL + el], a.cap);
                a.expertOffset[el] = off;
                a.expertCount[el] = min(totals[me * EL + el], a.cap - off);
            }
            if (threadIdx.x == 0) {
                const int last = me * EL + EL - 1;
                const int off = starts[last] + ((totals[last] + 127) & ~127);
                a.expertOffset[EL] = min(off, a.cap);
                if (off > a.cap) {
                    FailD(a.status, MF_DEV_ERR_BOUNDS);
                }
            }
        }
        __syncthreads();

        // ---- (c) quantise each token once, store it to the owners of its experts
        unsigned char *myStage = stage + (size_t)warp * stagePerWarp;
        uint32_t *myScale = reinterpret_cast<uint32_t *>(myStage + H);
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
                // Scale = smallest power of two >= amax / 448, as a biased exponent byte; multiplying by its reciprocal is exact.
                const uint32_t eb = Ue8m0Ceil(amax * (1.f / 448.f));
                const float inv = __uint_as_float((254u - eb) << 23);
                uint2 packed;
                unsigned short *ps = reinterpret_cast<unsigned short *>(&packed);
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    ps[i] = __nv_cvt_float2_to_fp8x2(make_float2(f[2 * i] * inv, f[2 * i + 1] * inv), __NV_SATFINITE, __NV_E4M3);
                }
                if (active) {
                    *reinterpret_cast<uint2 *>(myStage + off) = packed;
                    if ((lane & 15) == 0) {
                        myScale[blk] = eb * 0x01010101u;  // the same exponent for the four 32-element steps of the block
                    }
                }
            }
            __syncwarp();
            // Lane k owns pair (t, k): its row on the owner, and whether it leads the pairs of this token on that owner.
            int myE = -1, mySlot = -1, myOwner = -1;
            float myW = 0.f;
            if (lane < K) {
                myE = a.topkIdx[t * K + lane];
                myW = a.topkW[t * K + lane];
                if (myE >= 0 && myE < E) {
                    mySlot = sendBase[myE] + atomicAdd(&a.cursor[myE], 1);
                    myOwner = myE / EL;
                    if (mySlot >= a.cap) {
                        if (a.status != nullptr) {
                            atomicCAS(a.status, 0, MF_DEV_ERR_BOUNDS);
                        }
                        mySlot = -1;  // the owner's buffer is full: this pair is dropped and the call reports the overflow
                    }
                }
                if (a.sendSlot != nullptr) {
                    a.sendSlot[t * K + lane] = mySlot;
                }
            }
            // Pairs of one (token, owner) form groups of up to 1 + MF_MOE_MAX_SIBLINGS in k order; the first of a group leads it.
            int before = 0, nsib = 0;
            int2 sib[MF_MOE_MAX_SIBLINGS];
            for (int j = 0; j < K; j++) {
                const int oj = __shfl_sync(0xffffffffu, myOwner, j);
                const int sj = __shfl_sync(0xffffffffu, mySlot, j);
                const float wj = __shfl_sync(0xffffffffu, myW, j);
                if (mySlot >= 0 && sj >= 0 && oj == myOwner && j != lane) {
                    if (j < lane) {
                        before++;
                    } else if (nsib < MF_MOE_MAX_SIBLINGS) {
                        sib[nsib++] = make_int2(sj, __float_as_int(wj));
                    }
                }
            }
            const bool leader = mySlot >= 0 && before % (MF_MOE_MAX_SIBLINGS + 1) == 0;
            // In a large call only the leader of a (token, owner) group carries the payload over the link; the owner copies it
            // into the followers' rows after everything has landed (phase (e)): a token routed to several experts of one rank
            // crosses NVLink once.
            const uint32_t leadMask = __ballot_sync(0xffffffffu, leader);
            for (int k = 0; k < K; k++) {
                const int slot = __shfl_sync(0xffffffffu, mySlot, k);
                if (slot < 0 || (dedup && (leadMask >> k & 1u) == 0)) {
                    continue;
                }
                const uint32_t d = (uint32_t)__shfl_sync(0xffffffffu, myOwner, k);
                unsigned char *dx = reinterpret_cast<unsigned char *>(mf_shm_peer(m, a.recvX, d)) + (size_t)slot * H;
                uint32_t *ds = mf_shm_peer(m, a.recvSf, d) + (size_t)slot * nblk;
                for (int v = lane; v < H / 16; v += 32) {
                    mf_st16(dx + (size_t)v * 16, *reinterpret_cast<const uint4 *>(myStage + (size_t)v * 16));
                }
                for (int v = lane; v < nblk; v += 32) {
                    ds[v] = myScale[v];
                }
            }
            if (mySlot >= 0) {
                const uint32_t d = (uint32_t)myOwner;
                // Followers of a (token, owner) group are marked; the leader carries the number of siblings and their rows.
                const int kField = lane | (leader ? (nsib << 8) : MF_MOE_META_FOLLOWER);
                mf_shm_peer(m, a.recvMeta, d)[mySlot] = make_int4(me, t, kField, __float_as_int(myW));
                if (leader) {
                    int2 *sd = mf_shm_peer(m, a.recvSib, d) + (size_t)mySlot * MF_MOE_MAX_SIBLINGS;
                    for (int i = 0; i < nsib; i++) {
                        sd[i] = sib[i];
                    }
                }
            }
            if (arrival) {
                // Everything this warp stored for the token is visible system-wide before any of its rows is counted.
                __threadfence_system();
                __syncwarp();
                if (mySlot >= 0) {
                    atomicAdd_system(mf_shm_peer(m, a.arrive, (uint32_t)myOwner) + (mySlot >> 7), 1);
                }
            }
            __syncwarp();
        }
    }
    // ---- (d) everything I sent is visible before my arrival is; when all have arrived, all receive buffers are complete
    __threadfence_system();
    grid.sync();
    if (blockIdx.x == 0) {
        if (!dead && !arrival) {
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
    if (!dedup) {
        FinishEpochD(a, epochArg, epoch);
        return;  // every row came with its payload (in arrival mode the consumers wait on the tile counters)
    }
    // ---- (e) every leader row that arrived here is copied into the rows of its followers (local memory only)
    grid.sync();
    if (dead || ReadAbort(a.status, &abortFlag) != 0) {
        FinishEpochD(a, epochArg, epoch);
        return;
    }
    {
        const int warpsTotal = gridDim.x * kWarps;
        const int rowsHere = min(starts[me * EL + EL - 1] + ((totals[me * EL + EL - 1] + 127) & ~127), a.cap);
        const unsigned char *rx = reinterpret_cast<const unsigned char *>(a.recvX);
        for (int r = blockIdx.x * kWarps + warp; r < rowsHere; r += warpsTotal) {
            int el = 0;
            while (el + 1 < EL && starts[me * EL + el + 1] <= r) {
                el++;
            }
            if (r - starts[me * EL + el] >= totals[me * EL + el]) {
                continue;  // padding row: whatever it holds is from an earlier call
            }
            const int4 meta = mf_ld_meta(a.recvMeta + r);
            const int nsib = (meta.z >> 8) & 0xff;
            if ((meta.z & MF_MOE_META_FOLLOWER) != 0 || nsib == 0 || nsib > MF_MOE_MAX_SIBLINGS) {
                continue;
            }
            const int2 *sd = a.recvSib + (size_t)r * MF_MOE_MAX_SIBLINGS;
            int rowsOf[MF_MOE_MAX_SIBLINGS];
            int nf = 0;
            for (int i = 0; i < nsib; i++) {
                const int fr = sd[i].x;
                if (fr >= 0 && fr < rowsHere && fr != r) {
                    rowsOf[nf++] = fr;
                }
            }
            // The leader's row is read once, four vectors per lane at a time, and stored to every follower.
            const unsigned char *srcRow = rx + (size_t)r * H;
            for (int vb = lane; vb < H / 16; vb += 128) {
                uint4 raw[4];
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    raw[j] = vb + 32 * j < H / 16 ? mf_ld16_coherent(srcRow + (size_t)(vb + 32 * j) * 16) : make_uint4(0u, 0u, 0u, 0u);
                }
                for (int i = 0; i < nf; i++) {
                    unsigned char *dx = reinterpret_cast<unsigned char *>(a.recvX) + (size_t)rowsOf[i] * H;
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        if (vb + 32 * j < H / 16) {
                            mf_st16(dx + (size_t)(vb + 32 * j) * 16, raw[j]);
                        }
                    }
                }
            }
            for (int v = lane; v < nblk; v += 32) {
                const uint32_t w = ((volatile uint32_t *)a.recvSf)[(size_t)r * nblk + v];
                for (int i = 0; i < nf; i++) {
                    a.recvSf[(size_t)rowsOf[i] * nblk + v] = w;
                }
            }
        }
    }
    FinishEpochD(a, epochArg, epoch);
}

__global__ void __launch_bounds__(kThreads, 3)
mf_moe_combine_kernel(const mf_moe_combine_args_t *__restrict__ args, int H, int K, int EL, uint32_t channel, uint64_t epochArg, uint64_t timeoutNs)
{
    cg::grid_group grid = cg::this_grid();
    const mf_moe_combine_args_t a = args[blockIdx.y];
    const uint64_t epoch = ResolveEpochD(a, epochArg);
    if (epoch == 0) {
        FailD(a.status, MF_DEV_ERR_BOUNDS);  // neither an epoch argument nor a device-resident epoch
        return;
    }
    const MfDeviceMeta *m = reinterpret_cast<const MfDeviceMeta *>(a.meta);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int warpsTotal = gridDim.x * kWarps;
    __shared__ int offs[kMaxExperts + 1];
    __shared__ int cnts[kMaxExperts];
    __shared__ int abortFlag;
    if (mf_check_bounds_enabled(m) && !mf_shm_in_own_window(m, a.retY, (uint64_t)a.retRows * H * 2)) {
        FailD(a.status, MF_DEV_ERR_BOUNDS);
        FinishEpochD(a, epochArg, epoch);
        return;
    }
    for (int i = threadIdx.x; i <= EL; i += kThreads) {
        offs[i] = a.expertOffset[i];
        if (i < EL) {
            cnts[i] = a.expertCount[i];
        }
    }
    __syncthreads();
    const int rows = min(offs[EL], a.cap);
    const int vecs = H / 8;
    const uint32_t R = m->rankCount;
    // A call whose dispatch failed (overflow, timeout) moves no data; it still walks through the barriers so that the
    // peers' waits complete.
    const bool dead = ReadAbort(a.status, &abortFlag) != 0;

    // ---- push: one row per (token, owner): the leader's output plus its siblings', weighted, to the source rank's
    //      landing zone [token][k of the leader][:]
    // Work unit = (row, chunk of 128 vectors): a leader with many siblings is spread over several warps.
    const int chunks = (vecs + 127) / 128;
    for (long long u = (long long)blockIdx.x * kWarps + warp; u < (long long)rows * chunks && !dead; u += warpsTotal) {
        const int r = (int)(u / chunks), ch = (int)(u % chunks);
        int el = 0;
        while (el + 1 < EL && offs[el + 1] <= r) {
            el++;
        }
        if (r - offs[el] >= cnts[el]) {
            continue;  // padding row of the tile grid
        }
        const int4 meta = a.recvMeta[r];
        const uint32_t src = (uint32_t)meta.x;
        const int k = meta.z & 0xff, nsib = (meta.z >> 8) & 0xff;
        if ((meta.z & MF_MOE_META_FOLLOWER) != 0 || src >= R || meta.y < 0 || k >= K || (long long)meta.y * K + k >= a.retRows ||
            nsib > MF_MOE_MAX_SIBLINGS) {
            continue;
        }
        const int2 *sd = a.recvSib + (size_t)r * MF_MOE_MAX_SIBLINGS;
        int rowOf[MF_MOE_MAX_SIBLINGS + 1];
        float wOf[MF_MOE_MAX_SIBLINGS + 1];
        rowOf[0] = r;
        wOf[0] = __int_as_float(meta.w);
        int n = 1;
        for (int i = 0; i < nsib; i++) {
            const int2 e = sd[i];
            if (e.x >= 0 && e.x < rows) {
                rowOf[n] = e.x;
                wOf[n] = __int_as_float(e.y);
                n++;
            }
        }
        char *dst = reinterpret_cast<char *>(mf_shm_peer(m, a.retY, src)) + ((size_t)meta.y * K + k) * H * 2;
        // The lane's four vectors of the chunk are loaded together for every addend, so that four 16-byte loads per lane are
        // in flight (the rows of a group lie far apart: latency, not bandwidth, would pace a one-at-a-time loop).
        const int vEnd = min(vecs, (ch + 1) * 128);
        const int v0 = ch * 128 + lane;
        float acc[4][8];
#pragma unroll
        for (int j = 0; j < 4; j++) {
#pragma unroll
            for (int q = 0; q < 8; q++) {
                acc[j][q] = 0.f;
            }
        }
        for (int i = 0; i < n; i++) {
            const char *rowp = reinterpret_cast<const char *>(a.y) + (size_t)rowOf[i] * H * 2;
            uint4 raw[4];
#pragma unroll
            for (int j = 0; j < 4; j++) {
                raw[j] = v0 + 32 * j < vEnd ? mf_ld16(rowp + (size_t)(v0 + 32 * j) * 16) : make_uint4(0u, 0u, 0u, 0u);
            }
            const float w = wOf[i];
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const __nv_bfloat162 *h = reinterpret_cast<const __nv_bfloat162 *>(&raw[j]);
#pragma unroll
                for (int q = 0; q < 4; q++) {
                    float2 f = __bfloat1622float2(h[q]);
                    acc[j][2 * q] = fmaf(w, f.x, acc[j][2 * q]);
                    acc[j][2 * q + 1] = fmaf(w, f.y, acc[j][2 * q + 1]);
                }
            }
        }
#pragma unroll
        for (int j = 0; j < 4; j++) {
            if (v0 + 32 * j < vEnd) {
                uint4 pk;
                __nv_bfloat162 *hp = reinterpret_cast<__nv_bfloat162 *>(&pk);
#pragma unroll
                for (int q = 0; q < 4; q++) {
                    hp[q] = __floats2bfloat162_rn(acc[j][2 * q], acc[j][2 * q + 1]);
                }
                mf_st16(dst + (size_t)(v0 + 32 * j) * 16, pk);
            }
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
        FinishEpochD(a, epochArg, epoch);
        return;
    }
    // ---- add the owners' partial sums (fp32, fixed order): pair k carries one iff no earlier pair of the token has the same owner
    const int ELg = EL;
    for (int t = blockIdx.x * kWarps + warp; t < a.T; t += warpsTotal) {
        const char *base = reinterpret_cast<const char *>(a.retY) + (size_t)t * K * H * 2;
        char *o = reinterpret_cast<char *>(a.out) + (size_t)t * H * 2;
        uint32_t leaders = 0;
        for (int k = 0; k < K; k++) {
            const int e = a.topkIdx[t * K + k];
            if (e < 0 || e >= ELg * (int)R) {
                continue;
            }
            int before = 0;
            for (int j = 0; j < k; j++) {
                const int ej = a.topkIdx[t * K + j];
                if (ej >= 0 && ej < ELg * (int)R && ej / ELg == e / ELg) {
                    before++;
                }
            }
            if (before % (MF_MOE_MAX_SIBLINGS + 1) == 0) {
                leaders |= 1u << k;
            }
        }
        // Four vectors per lane and trip, loaded together for every partial sum (same reason as above).
        for (int vb = lane; vb < vecs; vb += 128) {
            float acc[4][8];
#pragma unroll
            for (int j = 0; j < 4; j++) {
#pragma unroll
                for (int q = 0; q < 8; q++) {
                    acc[j][q] = 0.f;
                }
            }
            for (int k = 0; k < K; k++) {
                if ((leaders >> k & 1u) == 0) {
                    continue;
                }
                const char *rowp = base + (size_t)k * H * 2;
                uint4 raw[4];
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    raw[j] = vb + 32 * j < vecs ? mf_ld16_coherent(rowp + (size_t)(vb + 32 * j) * 16) : make_uint4(0u, 0u, 0u, 0u);
                }
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const __nv_bfloat162 *h = reinterpret_cast<const __nv_bfloat162 *>(&raw[j]);
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        float2 f = __bfloat1622float2(h[i]);
                        acc[j][2 * i] += f.x;
                        acc[j][2 * i + 1] += f.y;
                    }
                }
            }
#pragma unroll
            for (int j = 0; j < 4; j++) {
                if (vb + 32 * j < vecs) {
                    uint4 pk;
                    __nv_bfloat162 *hp = reinterpret_cast<__nv_bfloat162 *>(&pk);
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        hp[i] = __floats2bfloat162_rn(acc[j][2 * i], acc[j][2 * i + 1]);
                    }
                    mf_st16(o + (size_t)(vb + 32 * j) * 16, pk);
                }
            }
        }
    }
    FinishEpochD(a, epochArg, epoch);
}

// Resident-CTA capacity of a kernel on the current device for a given dynamic shared-memory size; remembered per (device,
// kernel, size) because the occupancy query costs microseconds on a latency-critical call path.
int CoopCap(const void *kernel, size_t smem)
{
    struct Entry {
        const void *kernel;
        size_t smem;
        int dev;
        int capacity;
    };
    static Entry cache[32];
    static int used = 0;
    static std::mutex mu;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) {
        (void)cudaGetLastError();
        return 0;
    }
    {
        std::lock_guard<std::mutex> g(mu);
        for (int i = 0; i < used; i++) {
            if (cache[i].kernel == kernel && cache[i].smem == smem && cache[i].dev == dev) {
                return cache[i].capacity;
            }
        }
    }
    int perSm = 0, sms = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&perSm, kernel, kThreads, smem) != cudaSuccess) {
        (void)cudaGetLastError();
        return 0;
    }
    const int cap = perSm * sms;
    if (cap > 0) {
        std::lock_guard<std::mutex> g(mu);
        if (used < 32) {
            cache[used++] = Entry{kernel, smem, dev, cap};
        }
    }
    return cap;
}

}  // namespace

extern "C" int mf_k_moe_dispatch(const mf_moe_dispatch_args_t *argsDev, int nEmulatedRanks, int rankCount, int H, int K, int E, uint32_t channel,
                                 uint64_t epoch, uint64_t timeoutNs, int ctas, mf_stream_t stream)
{
    if (argsDev == nullptr || nEmulatedRanks < 1 || rankCount < 1 || rankCount > (int)MF_SIGNAL_MAX_RANKS || H <= 0 || H % 128 != 0 || K < 1 ||
        K > 32 || E < rankCount || E % rankCount != 0 || E > kMaxExperts || channel >= MF_SIGNAL_CHANNELS) {
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
        EL < 1 || EL > kMaxExperts || channel >= MF_SIGNAL_CHANNELS) {
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
