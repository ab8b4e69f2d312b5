/* Allreduce entry point that performs no allocation of any kind.
 *
 * This function has no counterpart in the reference; it exists for programs
 * that must not allocate device memory while they run: code whose whole memory
 * budget is handed to another allocator at start-up (a framework's caching
 * allocator, a fixed arena of a real-time service), where a stray cudaMalloc
 * can fail or fragment the budget, and code on latency-critical paths, where
 * cudaMalloc / cudaFree stall the whole device.  Such callers cannot create an
 * EmuWorld or a Communicator, both of which allocate an arena.
 *
 * What it does: the one-shot allreduce (sum, times `scale`) of `num_ranks`
 * float buffers that live on the CURRENT device, i.e. the single-GPU,
 * several-ranks form of the library's small-message kernel (every rank's CTAs
 * push their data into every other rank's slot, raise a flag, wait for the
 * others' flags with a bounded spin and add the copies in rank order).  The
 * slots and flags the kernel needs live in one file-scope device array that is
 * part of the library image:
 *
 *     limit  IBCOMM_NO_ALLOC_MAX_RANKS ranks (8), IBCOMM_NO_ALLOC_MAX_BYTES
 *            bytes per buffer (32 KiB = 8192 floats)
 *     cost   about 4.1 MiB of device memory on every GPU that loads the
 *            library, held until the process exits
 *
 * Larger requests are refused with code 1 and a message; nothing is launched.
 * The function calls no cudaMalloc, cudaFree or other allocating routine
 * (torch's included); the caller passes the inputs and the outputs.
 *
 * First call on a device: the address of the scratch array is looked up once
 * per device (with that device current) and remembered.  With CUDA's lazy
 * module loading (the default) the driver may also set the array up only at
 * that moment, which is work on the driver's side that can take time or fail:
 * make one warm-up call per device at start-up (or run with
 * CUDA_MODULE_LOADING=EAGER); the no-allocation guarantee holds from the
 * second call on.
 *
 * Stream capture: none of the calls may be made while `stream` is being
 * captured.  Every call ends by copying the kernel's error word to the host
 * and synchronising the stream, neither of which a capture allows.
 *
 * Threads: one process-wide lock is held for the whole call, the wait for the
 * kernel included, so calls from several threads run one after the other,
 * also when they target different GPUs.
 *
 * Sharing: every call on a device uses the same scratch array, which keeps
 * what the previous call left in it.  The flags are call counters that only
 * grow, so they need no clearing; the error word is cleared at the start of
 * every call.  Two calls that overlap on the GPU (different streams, different
 * threads) race on the slots: issue one at a time per device.
 *
 * The call enqueues its work on `stream` (0 = the null stream), waits for it
 * and returns 0, or 1 (bad argument / beyond the limits), 2 (a wait inside the
 * kernel ran out; the kernel returned normally), 3 (a CUDA call failed).
 * `errbuf` (may be NULL) receives a description of a failure.
 */
#pragma once

#include <stddef.h>

#define IBCOMM_NO_ALLOC_MAX_RANKS 8
#define IBCOMM_NO_ALLOC_MAX_BYTES (32 * 1024)

#ifdef __cplusplus
extern "C" {
#endif

int ibcomm_emu_oneshot_allreduce_f32_noalloc(const float* const* sendbufs, float* const* recvbufs, int num_ranks,
                                             size_t len_elements, float scale, void* stream, char* errbuf,
                                             size_t errbuf_len);

#ifdef __cplusplus
}
#endif
