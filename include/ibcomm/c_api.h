/* C interface of the library (for ctypes / FFI users; the PyTorch binding in
 * allreduce_proto_b200/ is built on it).  Every function returns 0 on success
 * or one of the library's error codes (1 invalid argument, 2 transport,
 * 3 CUDA, 4 not supported); ibcomm_last_error() then describes the failure.
 * Calling any function of this interface switches the library from
 * "exit on error" (the C++ default, like the reference) to "report".
 * The reference ships no binding (its README.md:62). */
#pragma once

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct ibcomm_comm ibcomm_comm;
typedef struct ibcomm_emu ibcomm_emu;

/* dtype: 0 float32, 1 float64, 2 int32, 3 int64, 4 float16, 5 bfloat16
 * algo : 0 auto, 1 ring, 2 rabenseifner, 3 nvls, 4 oneshot, 5 direct */

const char* ibcomm_last_error(void);
int ibcomm_has_cuda(void);

int ibcomm_create(int world_size, ibcomm_comm** out);
int ibcomm_destroy(ibcomm_comm* c);
int ibcomm_create_queue_pair(ibcomm_comm* c, int dest_rank, uint32_t info_out[3]);
int ibcomm_register_queue_pair(ibcomm_comm* c, int dest_rank, const uint32_t info[3]);
int ibcomm_register_process(ibcomm_comm* c, int dest_rank, const uint32_t info[3], uint32_t info_out[3]);
int ibcomm_register_myself(ibcomm_comm* c, int my_rank);
int ibcomm_set_timeout_ms(ibcomm_comm* c, int ms);
/* Upper bound of channels (CTAs) per collective; 0 restores IBCOMM_NUM_CUDA_STREAM. */
int ibcomm_set_max_channels(ibcomm_comm* c, int channels);

int ibcomm_send(ibcomm_comm* c, int dest_rank, const void* buf, size_t len, int blocking);
int ibcomm_recv(ibcomm_comm* c, int src_rank, void* buf, size_t len, int blocking);
int ibcomm_send_poll(ibcomm_comm* c, int dest_rank, int* done);
int ibcomm_recv_poll(ibcomm_comm* c, int src_rank, int* done);
int ibcomm_send_wait(ibcomm_comm* c, int dest_rank);
int ibcomm_recv_wait(ibcomm_comm* c, int src_rank);
int ibcomm_bcast(ibcomm_comm* c, void* buf, size_t len, int root);
int ibcomm_barrier(ibcomm_comm* c);

/* Host buffers: algo 1 (ring) or 2 (rabenseifner). */
int ibcomm_allreduce_host(ibcomm_comm* c, int algo, int dtype, const void* sendbuf, void* recvbuf, size_t len_elements);
/* Device buffers.  flags: bit 0 (IBCOMM_ASYNC) = only enqueue (ibcomm_check()
 * reports a failure after the caller synchronised), otherwise the call returns
 * when the result is in recvbuf; bit 1 (IBCOMM_USE_STREAM) = run on `stream`
 * taken literally (so the null stream can be named), otherwise on the
 * communicator's own stream. */
#define IBCOMM_ASYNC 1
#define IBCOMM_USE_STREAM 2
int ibcomm_allreduce_cuda(ibcomm_comm* c, int algo, int dtype, const void* sendbuf, void* recvbuf, size_t len_elements,
                          double scale, int wire_dtype, void* stream, int flags);
/* Host buffers: the halves of the ring allreduce (float32, float64, int32, int64). */
int ibcomm_reduce_scatter_host(ibcomm_comm* c, int dtype, const void* sendbuf, void* recvbuf, size_t block_elements);
int ibcomm_all_gather_host(ibcomm_comm* c, int dtype, const void* sendbuf, void* recvbuf, size_t block_elements);
/* Halves of the allreduce: block r belongs to rank r.  reduce_scatter: sendbuf
 * holds world_size blocks, recvbuf one; all_gather: the other way round.
 * algo: auto, nvls or direct. */
int ibcomm_reduce_scatter_cuda(ibcomm_comm* c, int algo, int dtype, const void* sendbuf, void* recvbuf, size_t block_elements,
                               double scale, void* stream, int flags);
int ibcomm_all_gather_cuda(ibcomm_comm* c, int algo, int dtype, const void* sendbuf, void* recvbuf, size_t block_elements,
                           void* stream, int flags);
int ibcomm_check(ibcomm_comm* c);
/* Which algorithm (codes of ibcomm_allreduce_cuda) and how many channels `auto`
 * takes for a device allreduce of `bytes`: nvls = multicast available and the
 * type has a switch reduction; mapped = both buffers mapped by the peers
 * (symmetric or registered memory).  Needs no GPU. */
int ibcomm_choose_algorithm(size_t bytes, int world_size, int nvls, int mapped, int max_channels, int* algo, int* channels);

/* Peer-mapped (and, with NVSwitch multicast, switch-reducible) device memory.
 * Collective: every rank calls with the same size in the same order. */
int ibcomm_symmetric_alloc(ibcomm_comm* c, size_t bytes, void** out);
int ibcomm_symmetric_free(ibcomm_comm* c, void* ptr);
/* Collective: maps a cudaMalloc'ed buffer of every rank (same size) into the
 * peers, so that allreduces on it skip the staging copies.  *id = -1 (on every
 * rank) when the memory cannot be shared; that is not an error. */
int ibcomm_register_buffer(ibcomm_comm* c, void* ptr, size_t bytes, int* id);
int ibcomm_deregister_buffer(ibcomm_comm* c, int id);

typedef struct {
  int device;
  int nvls;
  int share_mode;
  int last_algo;
  int last_channels;
  int pad_;
  uint64_t arena_bytes;
  uint64_t pool_bytes;
  uint64_t work_bytes;
  uint64_t calls;
  uint64_t kernel_launches;
  uint64_t switch_registrations; /* registered user buffers the switch kernels can use in place */
} ibcomm_device_info;
/* Connects the device path if necessary (collective on first use). */
int ibcomm_get_device_info(ibcomm_comm* c, int connect, ibcomm_device_info* out);

int ibcomm_set_timer_base(ibcomm_comm* c);
int ibcomm_dump_trace(ibcomm_comm* c);
/* Per-role stamps of the last traced call of the pipelined staged kernel (needs IBCOMM_TRACE=1): collects the
 * device trace, copies at most `capacity_words` words to `out` and stores the number available in `*words`
 * (8 x windows: pairs of nanoseconds from the first stamp; reducers, loader, storer, reducers' last store). */
int ibcomm_staged_timeline(ibcomm_comm* c, uint64_t* out, size_t capacity_words, size_t* words);

/* Several ranks emulated on one GPU (single cooperative launch per collective). */
int ibcomm_emu_create(int num_ranks, size_t pool_bytes, size_t work_bytes, ibcomm_emu** out);
int ibcomm_emu_destroy(ibcomm_emu* w);
int ibcomm_emu_allreduce(ibcomm_emu* w, int algo, int dtype, const void* const* sendbufs, void* const* recvbufs,
                         size_t len_elements, double scale, int wire_dtype, int channels, void* stream, int async);
int ibcomm_emu_set_timeout_ms(ibcomm_emu* w, int ms);
int ibcomm_emu_rsag(ibcomm_emu* w, int all_gather, int dtype, const void* const* sendbufs, void* const* recvbufs,
                    size_t block_elements, double scale, int channels, void* stream, int async);
int ibcomm_emu_last_channels(ibcomm_emu* w);
/* Test hook: rank `rank` does not take part in the following collectives
 * (-1 = everybody takes part), so its peers' bounded waits run out. */
int ibcomm_emu_set_silent_rank(ibcomm_emu* w, int rank);
/* Test hook: rank `rank` fails the executor's per-op bounds check (-1 = nobody);
 * no memory is touched out of range, the call reports "bad program". */
int ibcomm_emu_set_bad_program_rank(ibcomm_emu* w, int rank);
/* Direct algorithm: in place (0, default) or staged through the pool windows (1). */
int ibcomm_emu_set_direct_staging(ibcomm_emu* w, int on);
typedef struct {
  uint32_t code;
  uint32_t kind;
  int32_t rank;
  int32_t peer;
  int32_t channel;
  int32_t op_index;
  uint64_t expected;
  uint64_t seen;
  uint64_t seq;
} ibcomm_status_report;
int ibcomm_emu_last_status(ibcomm_emu* w, ibcomm_status_report* out);

/* out[i] = cast(in[i] * scale) on the current device. */
int ibcomm_copy_scale(const void* in, void* out, size_t len_elements, int dtype_in, int dtype_out, double scale, void* stream);

/* Utilities. */
int ibcomm_parse_number(const char* text, int64_t* out);

/* Named integer knobs of single kernels (include/ibcomm/tunables.h): a value set here wins over the environment
 * variable of the same name; value < 0 removes the override.  For tuning runs that sweep settings in one process. */
int ibcomm_set_tunable(const char* name, int value);
int ibcomm_get_tunable(const char* name, int dflt, int* out);
int ibcomm_get_exp_of_two(uint64_t n);
/* Writes up to `capacity` [begin, end) pairs; returns the count in *count. */
int ibcomm_split_buffer(size_t len_elements, size_t elem_bytes, size_t world_size, int64_t chunk_bytes, uint64_t* pairs,
                        size_t capacity, size_t* count);
int ibcomm_rank_to_chunk(size_t num_chunks, size_t world_size, int rank, int* chunks, size_t capacity, size_t* count);
/* Human-readable op program of one rank (for tests and debugging). */
int ibcomm_describe_program(int algo, int rank, int world_size, size_t len_elements, size_t elem_bytes, int64_t chunk_bytes,
                            size_t stage_bytes, char* text, size_t capacity);

#ifdef __cplusplus
}
#endif
