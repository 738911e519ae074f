/*
 * Big Memory (BM): a pool of HBM and host DRAM contributed by every rank, addressed through one Global Virtual Address
 * space, with memcpy-like xcopy between any two places of it.
 *
 * Counterpart of the reference's smem_bm.h / smem_bm_def.h (src/smem/include/host/smem_bm.h:28-197,
 * smem_bm_def.h:22-122); enum values and struct layouts match so that callers can switch by re-prefixing.
 * A pointer returned by mf_bm_ptr_by_mem_type(handle, type, peer) is base + peer * maxSize and is valid in every rank's
 * process and inside CUDA kernels of every rank.
 */
#ifndef MF_PUBLIC_MF_BM_H
#define MF_PUBLIC_MF_BM_H

#include "mf.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef void *mf_bm_t;
#define MF_BM_TIMEOUT_MAX UINT32_MAX
#define MF_BM_FLAG_NUMA_MASK 0x7FU          /* bits 0-6: NUMA node for the DRAM slice, 0x7F = the GPU's node */
#define MF_BM_FLAG_PERFORMANCE_MODE (1U << 7)
#define MF_BM_FLAG_CREATE_WITH_SHM (1U << 8) /* back the DRAM slice with the caller's dramShmFd */

typedef enum {
    MF_MEM_TYPE_LOCAL_DEVICE = 0,
    MF_MEM_TYPE_LOCAL_HOST,
    MF_MEM_TYPE_DEVICE, /* pooled HBM */
    MF_MEM_TYPE_HOST,   /* pooled DRAM */
    MF_MEM_TYPE_BUTT
} mf_bm_mem_type;

/* Which engines may move data. On B200: SDMA = copy kernels over NVLink with copy-engine fallback for host legs,
 * DEVICE_RDMA = the same kernels, HOST_* = CPU memcpy through the shared DRAM pool. */
typedef enum {
    MF_BM_DATA_OP_SDMA = 1U << 0,
    MF_BM_DATA_OP_HOST_RDMA = 1U << 1,
    MF_BM_DATA_OP_HOST_TCP = 1U << 2,
    MF_BM_DATA_OP_DEVICE_RDMA = 1U << 3,
    MF_BM_DATA_OP_HOST_URMA = 1U << 4,
    MF_BM_DATA_OP_BUTT
} mf_bm_data_op_type;

typedef enum {
    MF_BM_COPY_L2G = 0,  /* local HBM → pool */
    MF_BM_COPY_G2L = 1,  /* pool → local HBM */
    MF_BM_COPY_G2H = 2,  /* pool → local host memory */
    MF_BM_COPY_H2G = 3,  /* local host memory → pool */
    MF_BM_COPY_L2GH = 4, /* local HBM → pooled DRAM */
    MF_BM_COPY_GH2L = 5, /* pooled DRAM → local HBM */
    MF_BM_COPY_GH2H = 6, /* pooled DRAM → local host memory */
    MF_BM_COPY_H2GH = 7, /* local host memory → pooled DRAM */
    MF_BM_COPY_G2G = 8,  /* pool → pool */
    MF_BM_COPY_AUTO = 9, /* classify both pointers */
    MF_BM_COPY_BUTT
} mf_bm_copy_type;

typedef struct {
    uint32_t initTimeout;             /* seconds, default 120 */
    uint32_t createTimeout;           /* seconds, default 120 */
    uint32_t controlOperationTimeout; /* seconds, default 120 */
    bool startConfigStoreServer;      /* rank 0 (or the race winner under auto-ranking) hosts the store; default true */
    bool startConfigStoreOnly;        /* only host the store, create no pool */
    bool dynamicWorldSize;            /* ranks may join and leave */
    bool unifiedAddressSpace;         /* must be true */
    bool autoRanking;                 /* let the store hand out rank ids */
    uint16_t rankId;                  /* used when autoRanking is false */
    uint32_t flags;
    char hcomUrl[64];                 /* accepted for compatibility; unused inside one NVSwitch domain */
    mf_tls_config hcomTlsConfig;
    mf_tls_config storeTlsConfig;
} mf_bm_config_t;

typedef struct {
    uint64_t maxDramSize;   /* per-rank window of the DRAM pool (bytes, multiple of 2 MiB) */
    uint64_t maxHbmSize;    /* per-rank window of the HBM pool */
    uint64_t localDRAMSize; /* what this rank contributes (may be 0) */
    uint64_t localHBMSize;
    mf_bm_data_op_type dataOpType;
    uint32_t flags;
    char tag[32];
    char tagOpInfo[256]; /* "tagA:DEVICE_SDMA:tagB,tagA:HOST_RDMA:tagC" */
    int dramShmFd;
} mf_bm_create_option_t;

typedef struct {
    const void *src;
    void *dest;
    size_t dataSize;
} mf_copy_params;

typedef struct {
    void **sources;
    void **destinations;
    const uint64_t *dataSizes;
    uint32_t batchSize;
} mf_batch_copy_params;

int32_t mf_bm_config_init(mf_bm_config_t *config);
/* deviceId: CUDA device ordinal, or (uint16_t)MF_INVALID_DEV_ID for a CPU-only rank (DRAM pool only). */
int32_t mf_bm_init(const char *storeURL, uint32_t worldSize, uint16_t deviceId, const mf_bm_config_t *config);
void mf_bm_uninit(uint32_t flags);
uint32_t mf_bm_get_rank_id(void);
mf_bm_t mf_bm_create(uint32_t id, uint32_t memberSize, mf_bm_data_op_type dataOpType, uint64_t localDRAMSize, uint64_t localHBMSize,
                     uint32_t flags);
mf_bm_t mf_bm_create2(uint32_t id, const mf_bm_create_option_t *option);
void mf_bm_destroy(mf_bm_t handle);
int32_t mf_bm_join(mf_bm_t handle, uint32_t flags);
int32_t mf_bm_leave(mf_bm_t handle, uint32_t flags);
uint64_t mf_bm_get_local_mem_size_by_mem_type(mf_bm_t handle, mf_bm_mem_type memType);
void *mf_bm_ptr_by_mem_type(mf_bm_t handle, mf_bm_mem_type memType, uint16_t peerRankId);
int32_t mf_bm_copy(mf_bm_t handle, mf_copy_params *params, mf_bm_copy_type t, uint32_t flags);
int32_t mf_bm_copy_batch(mf_bm_t handle, mf_batch_copy_params *params, mf_bm_copy_type t, uint32_t flags);
/* Same as the two above but enqueued on the caller's CUDA stream (implies MF_ASYNC_COPY_FLAG). */
int32_t mf_bm_copy_on_stream(mf_bm_t handle, mf_copy_params *params, mf_bm_copy_type t, void *stream, uint32_t flags);
int32_t mf_bm_copy_batch_on_stream(mf_bm_t handle, mf_batch_copy_params *params, mf_bm_copy_type t, void *stream, uint32_t flags);
int32_t mf_bm_wait(mf_bm_t handle);
int32_t mf_bm_register_user_mem(mf_bm_t handle, uint64_t addr, uint64_t size);
int32_t mf_bm_unregister_user_mem(mf_bm_t handle, uint64_t addr);
uint32_t mf_bm_get_rank_id_by_gva(mf_bm_t handle, void *gva);
/* Number of ranks currently joined. */
uint32_t mf_bm_get_joined_size(mf_bm_t handle);

#ifdef __cplusplus
}
#endif
#endif
