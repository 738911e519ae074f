/*
 * Share Memory (SHM): a symmetric heap. Every rank contributes `symmetricSize` bytes of HBM; rank r's part lives at
 * gva + r * symmetricSize in every process and inside every rank's CUDA kernels, so device code reaches peers with plain
 * loads and stores over NVLink (see mf/device/mf_shm_device.cuh).
 *
 * Counterpart of the reference's smem_shm.h / smem_shm_def.h (src/smem/include/host/smem_shm.h:28-211,
 * smem_shm_def.h:21-47). Additions that a CUDA user needs and the reference keeps in fixed device addresses:
 * mf_shm_get_device_meta (the record device helpers read), the signal area used by device-side barriers, and the NVLS
 * multicast alias of the heap when the platform offers one.
 */
#ifndef MF_PUBLIC_MF_SHM_H
#define MF_PUBLIC_MF_SHM_H

#include "mf.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef void *mf_shm_t;
#define MF_SHM_EXTRA_CONTEXT_MAX 65536U
#define MF_SHM_SIGNAL_BYTES (2U * 1024U * 1024U) /* per-rank signal area, separate from the heap */

/* Engines a rank may use on the heap. MTE = loads/stores from kernels, SDMA = host-initiated copies, RDMA = NVLS multimem. */
typedef enum { MF_SHM_DATA_OP_MTE = 1U << 0, MF_SHM_DATA_OP_SDMA = 1U << 1, MF_SHM_DATA_OP_RDMA = 1U << 2 } mf_shm_data_op_type;

typedef struct {
    uint32_t shmInitTimeout;          /* seconds, default 120 */
    uint32_t shmCreateTimeout;        /* seconds, default 120 */
    uint32_t controlOperationTimeout; /* seconds, default 120 */
    bool startConfigStoreServer;      /* rank 0 hosts the store, default true */
    uint32_t flags;
} mf_shm_config_t;

int32_t mf_shm_config_init(mf_shm_config_t *config);
int32_t mf_shm_init(const char *configStoreIpPort, uint32_t worldSize, uint32_t rankId, uint16_t deviceId, mf_shm_config_t *config);
void mf_shm_uninit(uint32_t flags);
uint32_t mf_shm_query_support_data_operation(void);
/* Collective over [0, rankSize). symmetricSize: multiple of 2 MiB. On success *gva is rank 0's window start. */
mf_shm_t mf_shm_create(uint32_t id, uint32_t rankSize, uint32_t rankId, uint64_t symmetricSize, mf_shm_data_op_type dataOpType, uint32_t flags,
                       void **gva);
int32_t mf_shm_destroy(mf_shm_t handle, uint32_t flags);
int32_t mf_shm_set_extra_context(mf_shm_t handle, const void *context, uint32_t size);
uint32_t mf_shm_get_global_rank(mf_shm_t handle);
uint32_t mf_shm_get_global_rank_size(mf_shm_t handle);
int32_t mf_shm_control_barrier(mf_shm_t handle);
int32_t mf_shm_control_allgather(mf_shm_t handle, const char *sendBuf, uint32_t sendSize, char *recvBuf, uint32_t recvSize);
int32_t mf_shm_subgroup_barrier(mf_shm_t handle, const char *key, uint32_t rankSize, uint32_t rankId);
int32_t mf_shm_subgroup_allgather(mf_shm_t handle, const char *key, uint32_t rankSize, uint32_t rankId, const char *sendBuf, uint32_t sendSize,
                                  char *recvBuf, uint32_t recvSize);
/* reachInfo: bit mask of mf_shm_data_op_type usable towards remoteRank. */
int32_t mf_shm_topology_can_reach(mf_shm_t handle, uint32_t remoteRank, uint32_t *reachInfo);
int32_t mf_shm_atomic_alloc_value(mf_shm_t handle, uint32_t limit, uint32_t *value);
int32_t mf_shm_atomic_release_value(mf_shm_t handle, uint32_t value);
int32_t mf_shm_register_exit(mf_shm_t handle, void (*exitFn)(int));
int32_t mf_shm_global_exit(mf_shm_t handle, int status);

/* Device address of this object's 128-byte meta record (struct MfDeviceMeta in mf/device/mf_shm_device.cuh). */
const void *mf_shm_get_device_meta(mf_shm_t handle);
/* GVA of rank 0's signal area (rank r's is at + r * MF_SHM_SIGNAL_BYTES); zero-initialised, used by device barriers. */
void *mf_shm_get_signal_base(mf_shm_t handle);
/* NVLS multicast alias of the heap window of THIS rank's offset space (multimem.* addresses), or NULL if unavailable. */
void *mf_shm_get_multicast_ptr(mf_shm_t handle);
/* Next epoch value for device-side collectives on `channel` (0..MF_SHM_CHANNELS-1). All ranks must call in the same order. */
uint64_t mf_shm_next_epoch(mf_shm_t handle, uint32_t channel);
/* Debug switches read by device code (include/mf/device/mf_shm_device.cuh): bit 0 (MF_DEBUG_CHECK_BOUNDS) makes every library
 * kernel validate its heap arguments before it touches a peer and report MF_DEV_ERR_BOUNDS instead of accessing memory outside
 * the heap. Also switched on for every heap of the process by the environment variable MF_CHECK_BOUNDS=1. */
int32_t mf_shm_set_debug_flags(mf_shm_t handle, uint64_t flags);
#define MF_SHM_CHANNELS 16U

#ifdef __cplusplus
}
#endif
#endif
