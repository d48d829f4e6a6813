/**
 * @file noalloc.h
 * A single-GPU allreduce entry point that never allocates memory.
 *
 * This entry point has no counterpart in the reference library.  It exists for
 * callers that must not, or cannot, allocate device or pinned memory at the time
 * of the call: processes whose GPU memory has been handed over entirely to another
 * allocator (an inference server that reserves all HBM up front), clean-up paths
 * that run after an out-of-memory failure, and code under a "no allocation after
 * start-up" policy.  Every other entry point of the library creates a communicator
 * first, which allocates a workspace with cudaMalloc / cuMemCreate.
 *
 * What it does: the element-wise sum of `p` fp32 vectors that all live on the
 * current device (the same computation, with the same kernel and flag protocol,
 * as an allreduce over `p` emulated ranks), written to `p` output vectors.
 *
 * Where the scratch memory comes from: the staging slots and flags the kernel
 * needs live in one file-scope `static __device__` array of
 * AL_NOALLOC_SCRATCH_BYTES (about 4.2 MB) inside the library.  Every GPU that
 * loads the library holds that array until the process exits, whether or not this
 * function is ever called.
 *
 * Limits and rules:
 *  - 1 <= p <= AL_NOALLOC_MAX_RANKS and count <= AL_NOALLOC_MAX_COUNT; larger
 *    requests are rejected with an error, nothing is launched.
 *  - The first call on each device looks up the array's device address
 *    (cudaGetSymbolAddress) with that device current; make that first call before
 *    any stream capture begins.
 *  - All calls on a device share the one array, and it keeps what the previous call
 *    left in it.  Flags are epochs that only grow, so nothing needs clearing between
 *    calls, but two calls that overlap on the GPU (different streams, no ordering
 *    between them) race on the staging slots: order them yourself.
 *  - Inputs and outputs are the caller's; an output may alias its own rank's input.
 *  - No cudaMalloc, cudaFree, cudaHostAlloc or other allocating call is made.
 *  - Every wait inside the kernel is bounded (2 s).  If one runs out - which needs a GPU so
 *    oversubscribed that the cooperative grid's blocks stop making progress - the kernel
 *    marks the scratch as failed and returns without writing the outputs, and so does every
 *    later call: the launch itself still reports success, because the host never blocks.
 *    A caller that must know synchronises its stream and asks al_noalloc_status(); a
 *    non-zero code means the outputs of the calls since the last good status are not valid.
 *    al_noalloc_reset() clears the mark (and the whole array) once nothing is in flight.
 *
 * Returns 0 on success; otherwise non-zero and al_noalloc_last_error() describes
 * the problem (thread-local string, valid until the next call on this thread).
 */
#pragma once
#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

#define AL_NOALLOC_MAX_RANKS 8
#define AL_NOALLOC_MAX_COUNT 8192                       /* fp32 elements per rank */
#define AL_NOALLOC_SCRATCH_BYTES (8 * (4096 + 2 * 8 * 32768))

int al_noalloc_allreduce_f32(const float* const* inputs, float* const* outputs, int p, size_t count, void* stream);
/**
 * Reads the failure mark of the current device's scratch into *code: 0 = healthy, 1 = a wait
 * inside an earlier call ran out of time.  Copies a few words device-to-host with cudaMemcpy
 * into the caller's variable; allocates nothing.  Synchronise the streams you used first.
 */
int al_noalloc_status(int* code);
/**
 * Zeroes the scratch array of the current device on `stream` and restarts the epochs.  Call it
 * only when no al_noalloc_allreduce_f32 call is in flight on that device.  Allocates nothing.
 */
int al_noalloc_reset(void* stream);
const char* al_noalloc_last_error(void);

#ifdef __cplusplus
}
#endif
