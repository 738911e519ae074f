/*
 * Core memory-management and data-movement API, one level below BM / SHM / TRANS: entities, address-space reservation,
 * slices, export/import/map, and xcopy by explicit direction. Function-for-function counterpart of the reference's hybm C
 * API (src/hybm/include/hybm.h:28-57, hybm_big_mem.h:31-186, hybm_data_op.h:23-56, option struct hybm_def.h:36-141).
 * Typical order on every rank:
 *   mf_hybm_init → mf_hybm_create_entity → mf_hybm_reserve_mem_space → mf_hybm_alloc_local_memory → mf_hybm_export →
 *   (exchange the blobs by any means) → mf_hybm_import → mf_hybm_mmap → mf_hybm_data_copy ...
 */
#ifndef MF_PUBLIC_MF_HYBM_H
#define MF_PUBLIC_MF_HYBM_H

#include "mf.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef void *mf_hybm_entity_t;
typedef uint64_t mf_hybm_mem_slice_t;

#define MF_HYBM_FLAG_INIT_DEVICE_META (1ULL << 63)
#define MF_HYBM_FLAG_EXPORT_ENTITY (1U << 0)
#define MF_HYBM_EXCHANGE_DESC_MAX 512

enum { MF_BM_OK = 0, MF_BM_ERROR = -1, MF_BM_INVALID_PARAM = -2, MF_BM_MALLOC_FAILED = -3, MF_BM_NEW_OBJECT_FAILED = -4, MF_BM_TIMEOUT = -7,
       MF_BM_NOT_INITIALIZED = -9, MF_BM_NOT_SUPPORTED = -100 };

typedef enum { MF_HYBM_TYPE_KERNEL_INITIATE = 0, MF_HYBM_TYPE_HOST_INITIATE = 1 } mf_hybm_type;
typedef enum { MF_HYBM_MEM_TYPE_DEVICE = 1U << 0, MF_HYBM_MEM_TYPE_HOST = 1U << 1 } mf_hybm_mem_type;
/* Engines: KERNEL = load/store kernels (reference MTE), COPY_ENGINE = cudaMemcpyAsync (reference SDMA). */
typedef enum {
    MF_HYBM_DOP_KERNEL = 1U << 0,
    MF_HYBM_DOP_COPY_ENGINE = 1U << 1,
    MF_HYBM_DOP_DEVICE_RDMA = 1U << 2,
    MF_HYBM_DOP_HOST_RDMA = 1U << 3,
    MF_HYBM_DOP_HOST_TCP = 1U << 4,
    MF_HYBM_DOP_HOST_URMA = 1U << 5
} mf_hybm_data_op_type;
typedef enum { MF_HYBM_SCENE_DEFAULT = 0, MF_HYBM_SCENE_TRANS = 1, MF_HYBM_SCENE_SHM = 2 } mf_hybm_scene;
typedef enum { MF_HYBM_ROLE_PEER = 0, MF_HYBM_ROLE_SENDER = 1, MF_HYBM_ROLE_RECEIVER = 2 } mf_hybm_role;

/* L = local (outside the pool), G = global (pooled); H = host DRAM, D = device HBM. */
typedef enum {
    MF_HYBM_LH_TO_GH = 0, MF_HYBM_LH_TO_GD, MF_HYBM_LD_TO_GH, MF_HYBM_LD_TO_GD, MF_HYBM_GH_TO_LH, MF_HYBM_GH_TO_LD, MF_HYBM_GD_TO_LH,
    MF_HYBM_GD_TO_LD, MF_HYBM_GH_TO_GH, MF_HYBM_GH_TO_GD, MF_HYBM_GD_TO_GH, MF_HYBM_GD_TO_GD, MF_HYBM_DIRECTION_AUTO, MF_HYBM_DIRECTION_BUTT
} mf_hybm_copy_direction;

typedef struct {
    mf_hybm_type bmType;
    uint32_t memType;     /* mask of mf_hybm_mem_type */
    uint32_t bmDataOpType; /* mask of mf_hybm_data_op_type */
    mf_hybm_scene scene;
    mf_hybm_role role;
    uint32_t rankCount;
    uint32_t rankId;
    int32_t devId;        /* -1: CPU-only process */
    uint64_t maxHBMSize;  /* per-rank window of the HBM pool (multiple of 2 MiB) */
    uint64_t maxDRAMSize;
    uint64_t deviceVASpace; /* 0 = maxHBMSize */
    uint64_t hostVASpace;
    bool globalUniqueAddress;
    uint32_t flags;
    char transUrl[64];
    char tag[32];
    char tagOpInfo[256];
    int dramShmFd;
} mf_hybm_options;

typedef struct {
    uint8_t desc[MF_HYBM_EXCHANGE_DESC_MAX];
    uint32_t descLen;
} mf_hybm_exchange_info;

typedef struct {
    const void *src;
    void *dest;
    size_t dataSize;
} mf_hybm_copy_params;

typedef struct {
    void **sources;
    void **destinations;
    const uint64_t *dataSizes;
    uint32_t batchSize;
} mf_hybm_batch_copy_params;

int32_t mf_hybm_init(int32_t deviceId, uint64_t flags);
void mf_hybm_uninit(void);
int32_t mf_hybm_set_extern_logger(void (*logger)(int level, const char *msg));
int32_t mf_hybm_set_log_level(int level);
const char *mf_hybm_get_error_string(int32_t errCode);

mf_hybm_entity_t mf_hybm_create_entity(uint16_t id, const mf_hybm_options *options, uint32_t flags);
void mf_hybm_destroy_entity(mf_hybm_entity_t e, uint32_t flags);
/* hints: 0 = first free window; a rejected hint returns MF_BM_ERROR so that callers can negotiate a common address. */
int32_t mf_hybm_reserve_mem_space(mf_hybm_entity_t e, uint32_t flags);
int32_t mf_hybm_reserve_mem_space_at(mf_hybm_entity_t e, uint64_t hbmHint, uint64_t dramHint);
int32_t mf_hybm_unreserve_mem_space(mf_hybm_entity_t e, uint32_t flags);
void *mf_hybm_get_memory_ptr(mf_hybm_entity_t e, mf_hybm_mem_type memType);
mf_hybm_mem_slice_t mf_hybm_alloc_local_memory(mf_hybm_entity_t e, mf_hybm_mem_type memType, uint64_t size, uint32_t flags);
int32_t mf_hybm_free_local_memory(mf_hybm_entity_t e, mf_hybm_mem_slice_t slice, uint32_t flags);
void *mf_hybm_get_slice_va(mf_hybm_entity_t e, mf_hybm_mem_slice_t slice);
mf_hybm_mem_slice_t mf_hybm_register_local_memory(mf_hybm_entity_t e, const void *ptr, uint64_t size, uint32_t flags);
/* slice 0 (or MF_HYBM_FLAG_EXPORT_ENTITY) exports the entity record. */
int32_t mf_hybm_export(mf_hybm_entity_t e, mf_hybm_mem_slice_t slice, uint32_t flags, mf_hybm_exchange_info *exInfo);
int32_t mf_hybm_export_slice_size(mf_hybm_entity_t e, size_t *size);
int32_t mf_hybm_import(mf_hybm_entity_t e, const mf_hybm_exchange_info allExInfo[], uint32_t count, void *addresses[], uint32_t flags);
int32_t mf_hybm_mmap(mf_hybm_entity_t e, uint32_t flags);
int32_t mf_hybm_unmap(mf_hybm_entity_t e, uint32_t flags);
int32_t mf_hybm_remove_imported(mf_hybm_entity_t e, uint32_t rank, uint32_t flags);
int32_t mf_hybm_entity_reach_types(mf_hybm_entity_t e, uint32_t remoteRank, uint32_t *reachTypes, uint32_t flags);
int32_t mf_hybm_set_extra_context(mf_hybm_entity_t e, const void *context, uint32_t size);
const void *mf_hybm_get_device_meta(mf_hybm_entity_t e);

int32_t mf_hybm_data_copy(mf_hybm_entity_t e, mf_hybm_copy_params *params, mf_hybm_copy_direction direction, void *stream, uint32_t flags);
int32_t mf_hybm_data_batch_copy(mf_hybm_entity_t e, mf_hybm_batch_copy_params *params, mf_hybm_copy_direction direction, void *stream,
                                uint32_t flags);
int32_t mf_hybm_wait(mf_hybm_entity_t e);

#ifdef __cplusplus
}
#endif
#endif
