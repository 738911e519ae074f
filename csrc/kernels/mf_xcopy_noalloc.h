// Batch copy for callers that must not allocate device memory. This entry point has no counterpart in the reference
// library; it exists for embedders of this library.
//
// Who needs it: a serving engine that hands all of a GPU's free memory to its own pool at start-up leaves nothing for a
// later cudaMalloc, so a library call that allocates can fail long after the process looked healthy; and cudaMalloc /
// cudaFree synchronise the whole device, which a request path that is counted in microseconds cannot afford. The regular
// batch copy (mf_k_batch_xcopy) needs a device-resident copy of tables longer than 168 entries and gets it from
// cudaMalloc; this variant keeps that table, the chunk map and the completion counter in a fixed array that is part of
// the library image instead.
//
// Cost and limits: every GPU that loads the library holds the array (about 352 KiB) until the process exits, used or not.
// One call takes at most MF_NOALLOC_MAX_COPIES copies and MF_NOALLOC_MAX_CHUNKS chunks of 32 KiB (2 GiB of payload);
// larger batches are refused with MF_K_TOO_LARGE and a message on stderr — split them. Each copy is 1 byte .. 4 GiB-1.
//
// Sharing: all calls on a device use the same array. Calls are serialised on the host by a mutex, but the GPU work of two
// calls that were enqueued on different streams may overlap, and then the second table overwrites the first while it is
// still being read: enqueue such calls on one stream, or order the streams with events. The array keeps the last call's
// contents; each call zeroes the counter and rewrites the part of the table it uses, on the caller's stream.
//
// First call on a device: looks up the array's device address (cudaGetSymbolAddress, with that device current) and keeps it
// for later calls; an empty batch (count == 0) does just that, which makes it the warm-up call to issue during start-up,
// before any stream capture is begun on the device and before the embedder takes the remaining memory.
//
// Host-side cost: the table travels from ordinary (pageable) static host arrays with cudaMemcpyAsync. For tables up to
// roughly 64 KiB (about 2700 copies, or a chunk map of that size) the runtime stages the bytes and returns at once; beyond
// that it first waits until earlier work on `stream` has drained, so a very long table makes the call block the host.
// A call made while `stream` is being captured into a graph is refused with MF_K_INVALID: the staged table would be
// read again, with whatever a later call left there, every time the graph ran.
//
// The call never invokes cudaMalloc, cudaFree, or any allocating routine of the runtime, of this library or of torch; host
// side it uses only static storage. The caller passes inputs and outputs as device-visible addresses (local HBM, peer HBM
// mapped by this library, pinned host memory) in three host arrays, which may be reused as soon as the call returns.
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { MF_NOALLOC_MAX_COPIES = 4096, MF_NOALLOC_MAX_CHUNKS = 65536 };

// Enqueues `count` independent copies dsts[i] <- srcs[i] (sizes[i] bytes) as one kernel on `stream` (a cudaStream_t; NULL
// is the default stream). Returns 0, or MF_K_INVALID (-2) for bad arguments, MF_K_TOO_LARGE (-3) beyond the limits,
// MF_K_LAUNCH_FAILED (-1) if the runtime refused a step. Completion is the stream's: synchronise it or record an event.
int mf_batch_xcopy_noalloc(const uint64_t *srcs, const uint64_t *dsts, const uint64_t *sizes, uint32_t count, void *stream);

#ifdef __cplusplus
}
#endif
