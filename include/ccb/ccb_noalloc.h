/* An AllReduce entry point that allocates nothing. It has no counterpart in the
 * reference.
 *
 * Who needs it: code that is not allowed to call cudaMalloc (or anything that
 * allocates) at the point where it needs a collective. Examples are a plugin called
 * from inside a host application's latency-critical loop, where cudaMalloc would
 * serialise the whole device; a callback that runs while the application's own
 * caching allocator owns all free memory, so a foreign cudaMalloc can fail or
 * fragment it; and set-up-free tools that want to play a few ranks on one GPU
 * without creating a communicator (ccb_comm_create_local allocates one arena per
 * rank, a status word in pinned host memory and, for tracing, more).
 *
 * What it is: the same fused two-shot kernel as ccb_all_reduce on a local
 * communicator (all `nranks` ranks played on the current GPU by one cooperative
 * launch), but its staging arenas and flags live in a file-scope
 * `static __device__` array of CCB_NOALLOC_TOTAL_BYTES that is part of libccb.so's
 * image: every GPU on which the library is used holds that array until the process
 * exits. The caller still passes the input and output buffers.
 *
 * Rules:
 *  - The first call on a device looks the array's device address up and clears its
 *    flag words (a synchronous step). Make that first call before any stream capture
 *    is started on that device.
 *  - At most CCB_NOALLOC_MAX_RANKS ranks; the element count is limited by the array
 *    size: ask ccb_noalloc_max_count(). Larger requests fail with CCB_ERR_CAPACITY
 *    and a message in ccb_last_error(); nothing is launched.
 *  - All calls on a device share the one array and it keeps the previous call's
 *    contents; what must start from zero (the flags) is ordered by a call counter,
 *    not cleared. Two calls that overlap on the GPU (different streams, or different
 *    host threads without ordering) race on it: issue calls on one stream, or order
 *    them yourself.
 *  - A call returns CCB_OK once its kernel is launched. Every wait inside the kernel has
 *    a time limit (10 s); a wait that runs out makes the kernel return early and leaves
 *    `recv` partly written. That is NOT reported by the call that launched it: the
 *    kernel records it in status words inside the array, and ccb_noalloc_status() reads
 *    them back (a synchronising device-to-host copy of 32 bytes, no allocation). Call
 *    it where a synchronisation is affordable, e.g. once per step after the stream has
 *    been synchronised; a non-zero result means an earlier call's output must not be
 *    used. The ordinary entry points report the same event through ccb_comm_status().
 *  - No cudaMalloc, cudaFree, or allocating library routine is called, here or in
 *    anything these entry points call. */
#ifndef CCB_NOALLOC_H
#define CCB_NOALLOC_H

#include <stdint.h>

#include "ccb.h"

#ifdef __cplusplus
extern "C" {
#endif

#define CCB_NOALLOC_MAX_RANKS 4
#define CCB_NOALLOC_ARENA_BYTES (2u << 20) /* per rank: 1 MiB of flags + 1 MiB of staging */
#define CCB_NOALLOC_TOTAL_BYTES (CCB_NOALLOC_MAX_RANKS * CCB_NOALLOC_ARENA_BYTES)

/* Largest element count ccb_all_reduce_noalloc accepts for this shape (0 if the
 * shape itself is unsupported). */
uint64_t ccb_noalloc_max_count(int nranks, int dtype, int codec);

/* recv[r] = sum over r of send[r], r < nranks, all buffers on the current device;
 * `send` and `recv` are host arrays of nranks device pointers. Sum only. */
int ccb_all_reduce_noalloc(const void* const* send, void* const* recv, int nranks, uint64_t count, int dtype, int codec,
                           ccb_stream_t stream);

/* Status of the calls made so far on the current device: CCB_OK, or CCB_ERR_TIMEOUT
 * when a device-side wait of an earlier call gave up (then `words`, if not null,
 * receives the CCB_STATUS_WORDS status words: flags, where, epoch, last value seen).
 * Synchronises with the device. */
int ccb_noalloc_status(uint32_t* words);

#ifdef __cplusplus
}
#endif
#endif
