/*
 * memfabric-b200 public C API — common part.
 *
 * Function-for-function counterpart of the reference's smem.h (src/smem/include/host/smem.h:22-118): library
 * init/uninit, a standalone config-store server, logging control, TLS setters and the thread-local last-error text.
 * Names carry the prefix mf_ instead of smem_; include <mf/smem_compat.h> to keep compiling code written against the
 * reference's names. Error codes keep the reference's numeric values (src/smem/csrc/common/smem_types.h:22-37).
 */
#ifndef MF_PUBLIC_MF_H
#define MF_PUBLIC_MF_H

#include <stdbool.h>
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MF_ASYNC_COPY_FLAG (1UL << 0)  /* return after enqueueing; complete with *_wait() or the user's stream */
#define MF_COPY_KERNEL_FLAG (1UL << 1) /* force the load/store copy kernels (reference: COPY_EXTEND_FLAG) */
#define MF_WORLD_SIZE_MAX 1024U
#define MF_INVALID_DEV_ID (-1)         /* CPU-only process: no GPU is touched */

enum {
    MF_OK = 0,
    MF_ERROR = -1,
    MF_INVALID_PARAM = -2000,
    MF_MALLOC_FAILED = -2001,
    MF_NEW_OBJECT_FAILED = -2002,
    MF_NOT_STARTED = -2003,
    MF_TIMEOUT = -2004,
    MF_REPEAT_CALL = -2005,
    MF_DUPLICATED_OBJECT = -2006,
    MF_OBJECT_NOT_EXISTS = -2007,
    MF_NOT_INITIALIZED = -2008,
    MF_RESOURCE_IN_USE = -2009,
    MF_RECONNECT = -2010,
    MF_GET_OBJECT = -2011
};

#define MF_TLS_PATH_SIZE 256
typedef struct {
    bool tlsEnable;
    char caPath[MF_TLS_PATH_SIZE];
    char crlPath[MF_TLS_PATH_SIZE];
    char certPath[MF_TLS_PATH_SIZE];
    char keyPath[MF_TLS_PATH_SIZE];
    char keyPassPath[MF_TLS_PATH_SIZE];
    char packagePath[MF_TLS_PATH_SIZE];
    char decrypterLibPath[MF_TLS_PATH_SIZE];
} mf_tls_config;

typedef int (*mf_decrypt_handler)(const char *cipherText, size_t cipherTextLen, char *plainText, size_t *plainTextLen);

int32_t mf_init(uint32_t flags);
void mf_uninit(void);
/* Starts a config-store server in this process on tcp://ip:port (or tcp6://[ip]:port) and returns at once. */
int32_t mf_create_config_store(const char *storeUrl);
void mf_destroy_config_store(const char *storeUrl);
int32_t mf_set_extern_logger(void (*func)(int level, const char *msg));
int32_t mf_set_log_level(int level); /* 0 debug, 1 info, 2 warn, 3 error */
/* TLS 1.3 (mutual authentication) for every config-store link of the process. tlsInfo is the text form
 * "tlsCaPath: DIR; tlsCaFile: a.pem,b.pem; tlsCert: FILE; tlsCrlPath: DIR; tlsCrlFile: x.pem; packagePath: DIR" (tlsCert and
 * tlsCaFile are required; packagePath names the directory of libssl.so.3 when it is not the system's). The private key
 * (PEM text or the path of a PEM file) and its pass phrase (text or file; cipher text when a decrypt handler is given) are
 * registered with mf_set_config_store_tls_key. Both take effect for stores created afterwards. */
int32_t mf_set_conf_store_tls(bool enable, const char *tlsInfo, uint32_t tlsInfoLen);
int32_t mf_set_config_store_tls_key(const char *tlsPk, uint32_t tlsPkLen, const char *tlsPkPw, uint32_t tlsPkPwLen, mf_decrypt_handler h);
const char *mf_get_last_err_msg(void);
const char *mf_get_and_clear_last_err_msg(void);
const char *mf_version(void);

/* Aggregate tracer (count/min/max/avg per operation). dumpDir may be NULL: text is then only available via mf_trace_dump. */
int32_t mf_trace_enable(const char *dumpDir);
void mf_trace_disable(void);
/* Copies the current table as text into buf (truncated to len-1), returns the full length. */
size_t mf_trace_dump(char *buf, size_t len, bool reset);

#ifdef __cplusplus
}
#endif
#endif
