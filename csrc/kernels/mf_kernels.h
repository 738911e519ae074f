// Host-callable launchers of the library's CUDA kernels (C linkage, raw pointers and a cudaStream_t). Every launcher
// returns 0 on success or a negative code; nothing here synchronises unless stated.
#pragma once
#include <cstddef>
#include <cstdint>

#ifdef __CUDACC__
#include <vector_types.h>
#else
struct int4;  // only pointers to them cross this interface in host code
struct int2;
#endif

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CUstream_st *mf_stream_t;

enum { MF_K_OK = 0, MF_K_INVALID = -2, MF_K_LAUNCH_FAILED = -1, MF_K_TIMEOUT = -7, MF_K_TOO_LARGE = -3 };

// ------------------------------------------------------------------------------------------------ xcopy (K1 / K2)

// Single copy of n bytes between any two device-visible addresses (local HBM, peer HBM over NVLink, pinned host).
// ctas 0 = pick from the size.
int mf_k_xcopy(void *dst, const void *src, size_t n, int ctas, mf_stream_t stream);
int mf_k_xcopy_shaped(void *dst, const void *src, size_t n, uint32_t tile, uint32_t stages, uint32_t inflight, uint32_t blocked, int ctas,
                      mf_stream_t stream);

typedef struct {
    uint64_t src;
    uint64_t dst;
    uint32_t len;         // bytes, < 4 GiB (the host splits longer copies)
    uint32_t chunkStart;  // index of this descriptor's first chunk in the launch-wide chunk numbering
} mf_copy_desc_t;

enum { MF_BATCH_INLINE_MAX = 168, MF_BATCH_CHUNK_BYTES = 32768 };

// Batch of `count` independent copies in ONE launch. Descriptors must have chunkStart filled (prefix sum of
// ceil(len / MF_BATCH_CHUNK_BYTES)); totalChunks is the grand total. count <= MF_BATCH_INLINE_MAX travels in the kernel
// parameters; larger batches must pass `descsDev`, a device-readable copy of the table that is followed directly by
// uint32 map[totalChunks] giving each chunk's descriptor index. `doneCounter` (device, zero
// before first use, self-resetting) and `hostFlag` (pinned host word, may be NULL) implement completion signalling:
// the last CTA stores `flagValue` to *hostFlag with system-scope release semantics.
int mf_k_batch_xcopy(const mf_copy_desc_t *descs, const mf_copy_desc_t *descsDev, uint32_t count, uint32_t totalChunks,
                     uint32_t *doneCounter, volatile uint32_t *hostFlag, uint32_t flagValue, int ctas, mf_stream_t stream);

// ------------------------------------------------------------------------------------------------ allreduce + RMSNorm (K4)

// One block per (emulated) rank, resident in device memory. x must lie in the symmetric heap (peers read it at the same
// offset); residualOut must lie in the heap for the two-shot and NVLS algorithms (peers write it); the rest is local.
typedef struct {
    const void *meta;      // MfDeviceMeta of this rank (device pointer)
    const void *x;         // [T, H] bf16, this rank's addend
    const void *residual;  // [T, H] bf16 or NULL
    const void *weight;    // [H] bf16
    void *residualOut;     // [T, H] bf16: residual + sum_r x_r (may be NULL for one-shot)
    void *out;             // [T, H] bf16: RMSNorm(residualOut) * weight
    int *status;           // device int, zero before launch; receives MF_DEV_ERR_* | peer << 8 on a bounded-wait expiry
    // Device-resident epoch (optional): two 64-bit words, [0] = epoch of the last finished call, [1] = 0. With `epoch` 0 the
    // kernel takes epochState[0] + 1 as its epoch and the last CTA to finish stores it back, so the same launch can be
    // replayed from a CUDA graph (kernel arguments are frozen there, the epoch must still grow with every call).
    unsigned long long *epochState;
} mf_allreduce_args_t;

// MF_AR_ONESHOT_NOTAIL: one-shot without the closing cross-rank barrier. Only legal when the caller alternates between two x
// buffers from call to call: a rank then rewrites a buffer two calls later at the earliest, and by then every peer has passed
// the opening barrier of the call in between, i.e. has finished reading it.
enum { MF_AR_AUTO = 0, MF_AR_ONESHOT = 1, MF_AR_TWOSHOT = 2, MF_AR_NVLS = 3, MF_AR_ONESHOT_NOTAIL = 4 };

// argsDev: device array of nEmulatedRanks blocks (1 in production; R when a test runs all ranks of a fake heap on one GPU
// as slices of one cooperative launch). rankCount must equal meta->rankCount. epoch: strictly increasing per (heap,
// channel), identical on all ranks (mf_shm_next_epoch); 0 = take it from args->epochState (every rank must then do so, the
// states must have been initialised to the same value, at least the channel's last host-side epoch, and the channel must not
// be used with host-side epochs any more). H: multiple of 8, at most 16384. timeoutNs 0 = 2 s.
int mf_k_allreduce_rmsnorm(const mf_allreduce_args_t *argsDev, int nEmulatedRanks, int rankCount, int T, int H, float eps, int algo,
                           uint32_t channel, uint64_t epoch, uint64_t timeoutNs, int ctas, mf_stream_t stream);

// ------------------------------------------------------------------------------------------------ MoE expert FFN (K5b)

enum { MF_GEMM_EPI_BF16 = 0, MF_GEMM_EPI_SWIGLU = 1, MF_GEMM_EPI_SWIGLU_FP8 = 2 };
// OR-ed into `mode` of mf_k_moe_grouped_gemm_mx: the weights are pre-packed for streaming, b = [G][N/32][K/128][32][128] bytes
// (blocks of 32 rows x 128 K-bytes stored contiguously, 4 KiB each), so that a weight tile is read from DRAM in 4 KiB pieces
// instead of 128-byte pieces 'K' bytes apart. Same values, same result.
enum { MF_GEMM_B_PACKED = 1 << 8 };

// Grouped block-scaled FP8 GEMM on tcgen05 tensor cores. Group g owns rows [groupOffset[g], groupOffset[g] + groupCount[g])
// of A (group starts must be multiples of 128 rows; rows between count and the next start are ignored) and weights
// b[g] = [N, K]. a: [rowsTotal, K] e4m3, aScale: [rowsTotal, K/128] fp32, b: [G, N, K] e4m3, bScale: [G, N/128, K/128]
// fp32. out is bf16: [rowsTotal, N] for MF_GEMM_EPI_BF16; [rowsTotal, N/2] for MF_GEMM_EPI_SWIGLU, where every 64-row
// chunk of b[g] holds 32 gate rows followed by the 32 matching up rows and out = silu(gate) * up. N and K: multiples of 128.
// groupOffset/groupCount live on the device (the routing result never visits the host). status: device int or NULL.
int mf_k_moe_grouped_gemm(const void *a, const float *aScale, const void *b, const float *bScale, void *out, const int *groupOffset,
                          const int *groupCount, int G, int rowsTotal, int N, int K, int mode, int *status, int ctas, mf_stream_t stream);

// The same GEMM with the block scaling done by the tensor core (tcgen05.mma.kind::mxf8f6f4.block_scale): all scales are
// powers of two. aSf: [rowsTotal, K/128] 32-bit words, byte j of a word = UE8M0 exponent (value 2^(byte-127)) of K-elements
// [128*kb + 32*j, +32) of that row (a 1x128 scale is the same byte four times); bScale: [G, N/128, K/128] fp32 whose
// mantissa bits are ignored (only the exponent is used). Epilogues: MF_GEMM_EPI_BF16 (out bf16 [rowsTotal, N]),
// MF_GEMM_EPI_SWIGLU (out bf16 [rowsTotal, N/2]) and MF_GEMM_EPI_SWIGLU_FP8: out e4m3 [rowsTotal, N/2] plus outSf
// [rowsTotal, N/64] UE8M0 bytes, one per 32 outputs, i.e. exactly the a / aSf operands of a following GEMM with K = N/2.
// tileN: 0 = pick from the sizes; 128, 256 (N % 256 == 0), 224 (N % 224 == 0, bf16 epilogue only: two accumulators), or 512 =
// the two-SM kernel (256 x 256 tiles computed by pairs of CTAs with cta_group::2, N % 256 == 0; row-major weights only). a, b,
// out and aSf must be 16-byte aligned.
int mf_k_moe_grouped_gemm_mx(const void *a, const uint32_t *aSf, const void *b, const float *bScale, void *out, void *outSf,
                             const int *groupOffset, const int *groupCount, int G, int rowsTotal, int N, int K, int mode, int tileN,
                             int *status, int ctas, mf_stream_t stream);
// The same kernel driven by arrival counters: tile (group g, rows [off + 128 m, +128)) starts when arrive[(off + 128 m) / 128]
// has reached the number of valid rows of the tile (an acquire load of system scope, so what other GPUs stored into those
// rows before counting them is visible to the loads of the tile). waitNs bounds every such wait (0 = 2 s); on expiry *status
// becomes MF_K_GEMM_ARRIVAL_EXPIRED and the kernel drains and returns. A non-zero *status at launch (a failed dispatch) turns
// the waits off. tileN 512 is not available here.
enum { MF_K_GEMM_PIPELINE_EXPIRED = 3, MF_K_GEMM_ARRIVAL_EXPIRED = 4 };
int mf_k_moe_grouped_gemm_mx_gated(const void *a, const uint32_t *aSf, const void *b, const float *bScale, void *out, void *outSf,
                                   const int *groupOffset, const int *groupCount, int G, int rowsTotal, int N, int K, int mode, int tileN,
                                   const int *arrive, uint64_t waitNs, int *status, int ctas, mf_stream_t stream);
int mf_k_moe_grouped_gemm_mx_2sm(const void *a, const uint32_t *aSf, const void *b, const float *bScale, void *out, void *outSf,
                                 const int *groupOffset, const int *groupCount, int G, int rowsTotal, int N, int K, int mode, int *status, int ctas,
                                 mf_stream_t stream);

// ------------------------------------------------------------------------------------------------ MoE dispatch / combine (K5a, K5c)

// Per-rank argument blocks (device memory). "heap" fields must sit at the same offset of the symmetric heap on every rank.
typedef struct {
    const void *meta;     // MfDeviceMeta of this rank
    const void *x;        // [T, H] bf16 tokens of this rank
    const int *topkIdx;   // [T, K] global expert ids
    const float *topkW;   // [T, K] renormalised routing weights
    int *cnt;             // heap: [R][E] pair counts, row s written by rank s on every rank ([2][R][E] when `arrive` is set:
                          // calls alternate between the halves, since no closing barrier separates them)
    void *recvX;          // heap: [cap][H] e4m3
    uint32_t *recvSf;     // heap: [cap][H/128] scale words: the UE8M0 exponent byte of the 1x128 block, four times
    int4 *recvMeta;       // heap: [cap] {source rank, token, k | siblings << 8 | MF_MOE_META_FOLLOWER, weight bits}
    int2 *recvSib;        // heap: [cap][MF_MOE_MAX_SIBLINGS] {row, weight bits} of a leader's sibling rows
    int *localCnt;        // [E] scratch, zero before the first call (the kernel leaves it zero)
    int *cursor;          // [E] scratch, zero before the first call (the kernel leaves it zero)
    int *expertOffset;    // out: [E/R + 1] first row of each local expert (multiples of 128); last = rows in use
    int *expertCount;     // out: [E/R] valid rows of each local expert
    int *sendSlot;        // out (optional): [T, K] row each pair was written to on its owner
    int *status;          // device int, zero before launch
    int *arrive;          // heap, optional: [cap / 128] rows landed in each 128-row tile of the receive buffer (arrival mode: no
                          // closing barrier; the consumer waits per tile, see mf_k_moe_grouped_gemm_mx_gated). Between two
                          // dispatches in this mode a consumer must have waited for every tile of the first.
    unsigned long long *epochState;  // optional, [2] zero-initialised to {last finished epoch, 0}: with epoch argument 0 the kernel
                                     // takes its epoch from here and advances it itself, so launches can be replayed from a CUDA
                                     // graph. The same choice and the same starting epoch on every rank.
    int T;
    int cap;
    int dedupMinPairs;    // pairs per rank (average over the ranks) from which a token crosses the link once per owner and the owner
                          // replicates it; 0 = the built-in threshold. The same value on every rank.
    int reserved;
} mf_moe_dispatch_args_t;

// A token with several experts on one owner: the pair with the lowest k is the leader, the others are followers.
enum { MF_MOE_MAX_SIBLINGS = 7, MF_MOE_META_FOLLOWER = 1 << 30 };

typedef struct {
    const void *meta;
    const void *y;            // [cap][H] bf16 expert outputs (local)
    const int4 *recvMeta;     // as filled by dispatch (local side of the heap buffer)
    const int2 *recvSib;      // as filled by dispatch
    const int *expertOffset;  // as filled by dispatch
    const int *expertCount;
    void *retY;               // heap: [retRows][H] bf16 landing zone at the source rank, row = token * K + k
    const int *topkIdx;       // [T, K] as given to dispatch
    void *out;                // [T, H] bf16
    int *status;
    unsigned long long *epochState;  // optional: as in mf_moe_dispatch_args_t (a separate pair of words for this kernel)
    int T;
    int cap;                  // rows of the receive buffer (and of y)
    int retRows;              // rows of every rank's landing zone (max tokens * K)
    int reserved;
} mf_moe_combine_args_t;

// H: hidden (multiple of 128), K: experts per token, E: experts in total (multiple of the rank count). Both kernels are
// cooperative launches; epoch must grow by one per call and channel on every rank alike (epoch 0: taken from args.epochState).
int mf_k_moe_dispatch(const mf_moe_dispatch_args_t *argsDev, int nEmulatedRanks, int rankCount, int H, int K, int E, uint32_t channel,
                      uint64_t epoch, uint64_t timeoutNs, int ctas, mf_stream_t stream);
int mf_k_moe_combine(const mf_moe_combine_args_t *argsDev, int nEmulatedRanks, int rankCount, int H, int K, int EL, uint32_t channel,
                     uint64_t epoch, uint64_t timeoutNs, int ctas, mf_stream_t stream);

// ------------------------------------------------------------------------------------------------ weight reshard (K6)

// One destination sub-block: rows [r0, r0+nrows) x columns [c0, c0+ncols) of a row-major parameter with colsFull columns
// that starts at element srcFlatOff of the flat training vector. All of srcFlatOff, colsFull, c0 and ncols must be
// multiples of 8 elements. quant = 1 casts to e4m3 with one fp32 scale per 128x128 tile (nrows, ncols multiples of 128).
typedef struct {
    uint64_t srcFlatOff;
    uint64_t dstOff;    // BYTE offset of the sub-block in the destination buffer (row-major, ncols columns)
    uint64_t scaleOff;  // first scale of the sub-block in the scale buffer (floats), row-major over tiles
    uint32_t colsFull;
    uint32_t r0, c0;
    uint32_t nrows, ncols;
    uint32_t tileStart;  // prefix sum of ceil(nrows/128) * ceil(ncols/256) over the table (tiles are 128 rows x 256 columns)
    uint32_t quant;
    uint32_t pad;
} mf_reshard_desc_t;

typedef struct {
    const void *meta;
    const void *srcShard;  // heap: this rank's shard of the flat bf16 vector (same offset on every rank)
    void *dst;             // local destination buffer
    float *dstScale;       // local scale buffer (may be NULL if nothing is quantised)
    const mf_reshard_desc_t *descs;  // device table
    int *status;
    uint64_t shardElems;   // elements per shard (multiple of 8)
    uint32_t ndesc;
    uint32_t totalTiles;
} mf_reshard_args_t;

int mf_k_reshard(const mf_reshard_args_t *argsDev, int nEmulatedRanks, int rankCount, uint32_t channel, uint64_t epoch, uint64_t timeoutNs,
                 int ctas, mf_stream_t stream);

// bf16 [rows, K] → e4m3 [rows, K] + fp32 scales [rows, K/128] (scale = amax/448 per 128 elements). rowLimit (device int,
// may be NULL) caps the number of rows actually processed.
int mf_k_quant_rows_fp8(const void *x, void *q, float *scale, int rows, int K, const int *rowLimit, mf_stream_t stream);

// ------------------------------------------------------------------------------------------------ test support (K7)

// dst[i] = hash(seed, i) for i in [0, n) bytes; deterministic on host and device (see mf_k_pattern_byte_host).
int mf_k_fill_pattern(void *dst, size_t n, uint64_t seed, mf_stream_t stream);
// Counts bytes where buf[i] != hash(seed, i) into *mismatch (device-visible uint64, zeroed by the call).
int mf_k_check_pattern(const void *buf, size_t n, uint64_t seed, unsigned long long *mismatch, mf_stream_t stream);
// 64-bit order-independent checksum (sum of FNV-mixed 8-byte words, tail bytes zero-padded) into *out.
int mf_k_checksum(const void *buf, size_t n, unsigned long long *out, mf_stream_t stream);
unsigned char mf_k_pattern_byte_host(uint64_t seed, uint64_t index);
unsigned long long mf_k_checksum_host(const void *buf, size_t n);

// cudaMemcpyAsync(cudaMemcpyDefault) issued from inside the library (so that every CUDA call of a process that uses
// the bindings goes through one runtime instance). Returns the cudaError_t value.
int mf_k_memcpy_async(void *dst, const void *src, size_t n, mf_stream_t stream);

// SM count of the current device (cached per device), 0 without a GPU.
int mf_k_sm_count(void);

#ifdef __cplusplus
}
#endif
