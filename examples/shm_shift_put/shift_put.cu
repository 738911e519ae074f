// A user kernel on the symmetric heap: every rank puts a message into the next rank's heap with plain stores over NVLink,
// signals it, and waits (bounded) for the message of the previous rank. One process per GPU:
//     ./shift_put <rank> <world> tcp://127.0.0.1:7799
// (counterpart of the reference's example/shm/ShiftPutGet/shm_all_shift.cpp:86-141, with a wait that cannot hang)
#include <cstdio>
#include <cstdlib>
#include <cuda_runtime.h>

#include "mf/device/mf_shm_device.cuh"
#include "mf/mf.h"
#include "mf/mf_shm.h"

__global__ void ShiftPut(const MfDeviceMeta *meta, uint64_t epoch, int *status)
{
    const uint32_t me = mf_shm_get_global_rank(meta), n = mf_shm_get_global_rank_size(meta), next = (me + 1) % n, prev = (me + n - 1) % n;
    // message area: first 4 KiB of everybody's heap
    uint4 *dst = (uint4 *)mf_shm_ptr(meta, next, 0);
    for (uint32_t i = threadIdx.x; i < 256; i += blockDim.x) {
        mf_st16(dst + i, make_uint4(me, i, (uint32_t)epoch, 0xC0FFEE));
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        mf_quiet();                                                   // my stores before my signal
        mf_signal_set(mf_signal_ptr(meta, next, 1, 0, me), epoch);     // channel 1, slot 0
        if (!mf_wait_until_ge(mf_signal_ptr(meta, me, 1, 0, prev), epoch, 2000000000ull)) {
            *status = MF_DEV_ERR_TIMEOUT | (int)(prev << 8);
        }
    }
}

int main(int argc, char **argv)
{
    if (argc < 4) {
        fprintf(stderr, "usage: %s <rank> <world> <store-url>\n", argv[0]);
        return 2;
    }
    const int rank = atoi(argv[1]), world = atoi(argv[2]);
    cudaSetDevice(rank);
    mf_shm_config_t cfg;
    mf_shm_config_init(&cfg);
    if (mf_shm_init(argv[3], (uint32_t)world, (uint32_t)rank, (uint16_t)rank, &cfg) != MF_OK) {
        fprintf(stderr, "init failed: %s\n", mf_get_last_err_msg());
        return 1;
    }
    void *gva = nullptr;
    mf_shm_t shm = mf_shm_create(0, (uint32_t)world, (uint32_t)rank, 2u << 20, MF_SHM_DATA_OP_MTE, 0, &gva);
    if (shm == nullptr) {
        fprintf(stderr, "create failed: %s\n", mf_get_last_err_msg());
        return 1;
    }
    int *status = nullptr;
    cudaMallocManaged(&status, sizeof(int));
    *status = 0;
    ShiftPut<<<1, 256>>>((const MfDeviceMeta *)mf_shm_get_device_meta(shm), mf_shm_next_epoch(shm, 1), status);
    cudaError_t e = cudaDeviceSynchronize();
    uint32_t first[4] = {0};
    cudaMemcpy(first, (char *)gva + (size_t)rank * (2u << 20), sizeof(first), cudaMemcpyDeviceToHost);
    printf("rank %d: cuda=%d status=%d message from rank %u (tag %x)\n", rank, (int)e, *status, first[0], first[3]);
    mf_shm_control_barrier(shm);
    int ok = e == cudaSuccess && *status == 0 && first[0] == (uint32_t)((rank + world - 1) % world) && first[3] == 0xC0FFEE;
    mf_shm_destroy(shm, 0);
    mf_shm_uninit(0);
    return ok ? 0 : 1;
}
