/*
 * Transfer engine (TRANS): one-sided read/write between processes that register arbitrary buffers — the building block for
 * prefill/decode KV-cache transfer. No pool and no common address: a peer is named by its unique id ("ip:port" string) and
 * its memory by the address it has in the peer's own process.
 *
 * Counterpart of the reference's smem_trans.h / smem_trans_def.h (src/smem/include/host/smem_trans.h:30-239,
 * smem_trans_def.h:22-45). Differences that a caller can see: registration is effective as soon as the call returns (the
 * reference sleeps 8 s after registering, src/smem/csrc/smem_trans/smem_trans.cpp:124-125); a peer's registrations are
 * fetched from the store on first use and whenever an address is not yet known, instead of by a 3-second polling thread.
 */
#ifndef MF_PUBLIC_MF_TRANS_H
#define MF_PUBLIC_MF_TRANS_H

#include "mf.h"
#include "mf_bm.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef void *mf_trans_t;

typedef enum { MF_TRANS_NONE = 0, MF_TRANS_SENDER, MF_TRANS_RECEIVER, MF_TRANS_BOTH, MF_TRANS_BUTT } mf_trans_role_t;

typedef struct {
    mf_trans_role_t role;
    uint32_t initTimeout; /* seconds, default 120 */
    uint32_t deviceId;    /* CUDA device ordinal */
    uint32_t flags;
    mf_bm_data_op_type dataOpType; /* default SDMA: copy kernels over NVLink */
    bool startConfigServer;        /* host the store in this process (default false) */
} mf_trans_config_t;

int32_t mf_trans_config_init(mf_trans_config_t *config);
int32_t mf_trans_init(const mf_trans_config_t *config);
void mf_trans_uninit(uint32_t flags);
mf_trans_t mf_trans_create(const char *storeUrl, const char *uniqueId, const mf_trans_config_t *config);
int32_t mf_trans_destroy(mf_trans_t handle, uint32_t flags);

/* Pinned host memory that peers can map (backed by an anonymous shared file). */
void *mf_trans_malloc(mf_trans_t handle, size_t capacity);
int32_t mf_trans_free(mf_trans_t handle, void *address);

/* Makes [address, address + capacity) readable and writable by peers. Device memory from cudaMalloc / torch, device memory
 * created with the CUDA VMM API, and memory returned by mf_trans_malloc can be registered. */
int32_t mf_trans_register_mem(mf_trans_t handle, void *address, size_t capacity, uint32_t flags);
int32_t mf_trans_batch_register_mem(mf_trans_t handle, void *addresses[], size_t capacities[], uint32_t count, uint32_t flags);
int32_t mf_trans_deregister_mem(mf_trans_t handle, void *address);

/* Synchronous one-sided transfers. remoteAddr is an address inside a range the peer registered, in the peer's terms. */
int32_t mf_trans_write(mf_trans_t handle, const void *localAddr, const char *remoteUniqueId, void *remoteAddr, size_t dataSize, uint32_t flags);
int32_t mf_trans_read(mf_trans_t handle, void *localAddr, const char *remoteUniqueId, const void *remoteAddr, size_t dataSize, uint32_t flags);
int32_t mf_trans_batch_write(mf_trans_t handle, const void *localAddrs[], const char *remoteUniqueId, void *remoteAddrs[], size_t dataSizes[],
                             uint32_t batchSize, uint32_t flags);
int32_t mf_trans_batch_read(mf_trans_t handle, void *localAddrs[], const char *remoteUniqueId, const void *remoteAddrs[], size_t dataSizes[],
                            uint32_t batchSize, uint32_t flags);
/* The same, enqueued on the caller's CUDA stream (NULL = the default stream); completion is the stream's business. */
int32_t mf_trans_write_submit(mf_trans_t handle, const void *localAddr, const char *remoteUniqueId, void *remoteAddr, size_t dataSize, void *stream,
                              uint32_t flags);
int32_t mf_trans_read_submit(mf_trans_t handle, void *localAddr, const char *remoteUniqueId, const void *remoteAddr, size_t dataSize, void *stream,
                             uint32_t flags);
int32_t mf_trans_batch_write_submit(mf_trans_t handle, const void *localAddrs[], const char *remoteUniqueId, void *remoteAddrs[],
                                    size_t dataSizes[], uint32_t batchSize, void *stream, uint32_t flags);
int32_t mf_trans_batch_read_submit(mf_trans_t handle, void *localAddrs[], const char *remoteUniqueId, const void *remoteAddrs[], size_t dataSizes[],
                                   uint32_t batchSize, void *stream, uint32_t flags);
/* Rank id the store assigned to this engine (stable across a reconnect; reused ids are handed out after a peer died). */
uint32_t mf_trans_get_rank(mf_trans_t handle);

#ifdef __cplusplus
}
#endif
#endif
