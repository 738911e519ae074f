// Device-initiated one-sided operations on the symmetric heap, measured from inside the kernels: put + signal ping-pong latency
// between two ranks, and put / get bandwidth of one rank into / out of its neighbour's heap, for message sizes 16 B - 4 MiB.
// One process per GPU, two ranks:
//     ./put_signal_bench <rank> 2 tcp://127.0.0.1:7801
// Every wait in the kernels is bounded (2 s): if the other rank never shows up the kernel records a time-out status and
// returns, the program prints it and exits non-zero. Counterpart of the reference's device-side RDMA demo
// (example/shm/RDMADemo/shm_rdma_test_dev.cpp:25-98: write test, read test and completion polling issued from a kernel), with
// NVLink stores/loads in place of work requests and a release/acquire flag in place of the completion queue.
#include <cstdio>
#include <cstdlib>
#include <cuda_runtime.h>

#include "mf/device/mf_shm_device.cuh"
#include "mf/mf.h"
#include "mf/mf_shm.h"

constexpr uint64_t kWaitNs = 2000000000ull;
constexpr uint32_t kHeapBytes = 16u << 20;
constexpr uint32_t kMsgOff = 0;             // message area of every heap: [0, 4 MiB)
constexpr uint32_t kSrcOff = 8u << 20;      // local source / destination area: [8 MiB, 12 MiB)

struct Result {
    int status;
    int pad;
    unsigned long long ns;
};

// Ping-pong: rank 0 puts `bytes` into rank 1 and raises rank 1's flag; rank 1 waits for it, puts `bytes` back and raises rank
// 0's flag; `iters` round trips. One CTA per rank. Half the round-trip time is the one-way put+signal latency.
__global__ void PingPong(const MfDeviceMeta *meta, uint64_t epochBase, uint32_t bytes, uint32_t iters, Result *res)
{
    const uint32_t me = mf_shm_get_global_rank(meta), peer = 1 - me;
    char *remote = (char *)mf_shm_ptr(meta, peer, kMsgOff);
    const char *local = (const char *)mf_shm_ptr(meta, me, kSrcOff);
    uint64_t *peerFlag = mf_signal_ptr(meta, peer, 2, 0, me);
    const uint64_t *myFlag = mf_signal_ptr(meta, me, 2, 0, peer);
    __shared__ int failed;
    if (threadIdx.x == 0) {
        failed = 0;
    }
    __syncthreads();
    const uint64_t t0 = mf_globaltimer_ns();
    for (uint32_t i = 0; i < iters && !failed; i++) {
        const uint64_t e = epochBase + i;
        if (me == 0) {
            mf_put16(remote, local, bytes);
            __syncthreads();
            if (threadIdx.x == 0) {
                mf_quiet();
                mf_signal_set(peerFlag, e);
                if (!mf_wait_until_ge(myFlag, e, kWaitNs)) {
                    failed = 1;
                }
            }
            __syncthreads();
        } else {
            if (threadIdx.x == 0 && !mf_wait_until_ge(myFlag, e, kWaitNs)) {
                failed = 1;
            }
            __syncthreads();
            if (!failed) {
                mf_put16(remote, local, bytes);
                __syncthreads();
                if (threadIdx.x == 0) {
                    mf_quiet();
                    mf_signal_set(peerFlag, e);
                }
            }
        }
    }
    if (threadIdx.x == 0) {
        res->ns = mf_globaltimer_ns() - t0;
        res->status = failed ? MF_DEV_ERR_TIMEOUT : 0;
    }
}

// Bandwidth: every CTA moves its share of `bytes` `iters` times, put (stores to the peer) or get (loads from the peer).
__global__ void Stream(const MfDeviceMeta *meta, uint32_t bytes, uint32_t iters, int get, Result *res)
{
    const uint32_t me = mf_shm_get_global_rank(meta), peer = 1 - me;
    const uint32_t share = (bytes / gridDim.x) & ~15u;
    char *remote = (char *)mf_shm_ptr(meta, peer, kMsgOff) + (size_t)blockIdx.x * share;
    char *local = (char *)mf_shm_ptr(meta, me, kSrcOff) + (size_t)blockIdx.x * share;
    const uint64_t t0 = mf_globaltimer_ns();
    for (uint32_t i = 0; i < iters; i++) {
        if (get) {
            mf_get16(local, remote, share);
        } else {
            mf_put16(remote, local, share);
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        mf_quiet();
        atomicMax(&res->ns, mf_globaltimer_ns() - t0);
    }
}

#define CHECK_CUDA(x)                                                                    \
    do {                                                                                 \
        cudaError_t e_ = (x);                                                            \
        if (e_ != cudaSuccess) {                                                         \
            fprintf(stderr, "%s failed: %s\n", #x, cudaGetErrorString(e_));              \
            return 1;                                                                    \
        }                                                                                \
    } while (0)

int main(int argc, char **argv)
{
    if (argc < 4) {
        fprintf(stderr, "usage: %s <rank> 2 <store-url>\n", argv[0]);
        return 2;
    }
    const int rank = atoi(argv[1]), world = atoi(argv[2]);
    if (world != 2 || rank < 0 || rank > 1) {
        fprintf(stderr, "this benchmark runs on exactly two ranks\n");
        return 2;
    }
    CHECK_CUDA(cudaSetDevice(rank));
    mf_shm_config_t cfg;
    mf_shm_config_init(&cfg);
    if (mf_shm_init(argv[3], 2, (uint32_t)rank, (uint16_t)rank, &cfg) != MF_OK) {
        fprintf(stderr, "init failed: %s\n", mf_get_last_err_msg());
        return 1;
    }
    void *gva = nullptr;
    mf_shm_t shm = mf_shm_create(0, 2, (uint32_t)rank, kHeapBytes, MF_SHM_DATA_OP_MTE, 0, &gva);
    if (shm == nullptr) {
        fprintf(stderr, "create failed: %s\n", mf_get_last_err_msg());
        return 1;
    }
    const MfDeviceMeta *meta = (const MfDeviceMeta *)mf_shm_get_device_meta(shm);
    Result *res = nullptr;
    CHECK_CUDA(cudaMallocManaged(&res, sizeof(Result)));
    int rc = 0;
    if (rank == 0) {
        printf("%10s %16s %14s %14s\n", "bytes", "put+signal us", "put GB/s", "get GB/s");
    }
    const uint32_t iters = 200;
    for (uint32_t bytes = 16; bytes <= (4u << 20) && rc == 0; bytes *= 4) {
        // latency: both ranks run the ping-pong at the same time (each on its own GPU)
        *res = Result{0, 0, 0};
        uint64_t epoch = 0;
        for (uint32_t i = 0; i < iters; i++) {
            epoch = mf_shm_next_epoch(shm, 2);  // one epoch per round trip; the kernel uses epochBase + i
        }
        const uint64_t base = epoch - iters + 1;
        mf_shm_control_barrier(shm);
        PingPong<<<1, 256>>>(meta, base, bytes, iters, res);
        CHECK_CUDA(cudaDeviceSynchronize());
        if (res->status != 0) {
            fprintf(stderr, "rank %d: ping-pong of %u bytes timed out (status %d)\n", rank, bytes, res->status);
            rc = 1;
            break;
        }
        const double latUs = (double)res->ns / iters / 2.0 / 1e3;
        // bandwidth: rank 0 streams while rank 1 idles (its memory is the target)
        double putGb = 0, getGb = 0;
        mf_shm_control_barrier(shm);
        if (rank == 0) {
            const int ctas = bytes >= (64u << 10) ? 64 : 1;
            for (int get = 0; get < 2; get++) {
                *res = Result{0, 0, 0};
                Stream<<<ctas, 512>>>(meta, bytes, iters, get, res);
                CHECK_CUDA(cudaDeviceSynchronize());
                const double gb = (double)((bytes / ctas) & ~15u) * ctas * iters / (double)res->ns;
                (get ? getGb : putGb) = gb;
            }
            printf("%10u %16.2f %14.2f %14.2f\n", bytes, latUs, putGb, getGb);
        }
        mf_shm_control_barrier(shm);
    }
    mf_shm_control_barrier(shm);
    cudaFree(res);
    mf_shm_destroy(shm, 0);
    mf_shm_uninit(0);
    return rc;
}
