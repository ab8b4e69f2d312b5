// Host-callable launchers of the device kernels (one translation unit each).
#pragma once

#include <cuda_runtime.h>

#include "ibcomm/communicator.h"
#include "ibcomm/device_types.h"

namespace ibcomm {

// ---- op-program executor (ring, Rabenseifner) ----
// `emu` == nullptr: one rank, grid = channels.  Otherwise `emu` points to
// `emu_ranks` parameter blocks in device memory and the launch is cooperative.
cudaError_t LaunchExecKernel(const ExecParams& p, const ExecParams* emu, int emu_ranks, int channels, cudaStream_t stream);
// CTA size the executor uses for a grid of `channels` CTAs, and the largest
// grid of CTAs of `threads` threads (0 = the full-size CTA) that is co-resident
// on `device` (0 on error).  CTA b of a rank waits for CTA b of the other
// ranks, so a collective never launches more CTAs than fit at once.
int ExecKernelThreadsFor(int channels);
int ExecKernelMaxCoResidentBlocks(int device, int threads = 0);

// ---- world_size == 1, and local staging: out = cast(in * scale) ----
// Uses bulk asynchronous copies (TMA, non-tensor form) through shared memory.
struct CopyParams {
  const void* in;
  void* out;
  uint64_t len_elements;
  int32_t dtype_in;
  int32_t dtype_out;
  double scale;
};
// Eight CTAs per SM of a B200 (one resident at a time, the rest queued): the
// hardware scheduler then overlaps the tail of one launch with the head of
// the next, which a one-CTA-per-SM persistent grid cannot (measured: 6.38 TB/s
// read+write against 5.81 TB/s).
constexpr int kCopyDefaultBlocks = 148 * 8;
cudaError_t LaunchCopyKernel(const CopyParams& p, int blocks, cudaStream_t stream);

// ---- two-shot allreduce: in the NVSwitch (multimem) or by direct peer loads/stores ----
struct NvlsParams {
  int32_t rank;
  int32_t world_size;
  int32_t dtype;
  int32_t use_multimem;  // 1: multimem.ld_reduce / multimem.st; 0: peer loads + peer stores
  int32_t stage_in;    // copy sendbuf into the multicast-bound staging first
  int32_t stage_out;   // results land in staging and are copied to recvbuf
  PeerTable peers;     // control pages live in the arenas
  const void* sendbuf;
  void* recvbuf;
  uint64_t len_elements;
  double scale;
  // Multicast and local addresses of the input and output windows.  When
  // staged, a window holds `window_elems` elements and the message is
  // processed in rounds; when zero-copy, the window is the whole buffer.
  unsigned char* mc_in;
  unsigned char* mc_out;
  unsigned char* local_in;
  unsigned char* local_out;
  // Unicast views of every rank's input window (direct variant; unaligned tail)
  // and output window (direct variant).
  unsigned char* peer_in[kMaxRanks];
  unsigned char* peer_out[kMaxRanks];
  uint64_t window_elems;
  // Staged input only: byte offset (from local_in / peer_in) of the 16 bytes
  // that hold the ragged end of the message, outside every window, so that
  // CTA 0, which moves the ragged end, touches no bytes that belong to another
  // CTA's part of a window.
  uint64_t tail_in_off;
  uint64_t timeout_ns;
  DeviceStatus* status;
  uint32_t* doorbell;
};
cudaError_t LaunchNvlsKernel(const NvlsParams& p, const NvlsParams* emu, int emu_ranks, int blocks, cudaStream_t stream);
// Largest co-resident grid of the two-shot kernels (they share CTA size and register budget).
int TwoShotKernelMaxCoResidentBlocks(int device);

// Hybrid two-shot (hybrid_kernel.cu): zero-copy symmetric buffers; CTAs
// [0, nvls_ctas) reduce 16-byte vectors [0, split_vec) in the switch, the other
// CTAs of the grid reduce the rest with peer loads and stores.
struct HybridParams {
  NvlsParams base;
  int32_t nvls_ctas;
  int32_t pad_;
  uint64_t split_vec;
};
cudaError_t LaunchHybridKernel(const HybridParams& h, int blocks, cudaStream_t stream);

// ---- pipelined staged two-shot (staged_kernel.cu) ----
// For buffers the peers cannot map, and for fp32 buffers that travel as
// bf16/fp16: the message moves through the pool in windows, and inside one
// CTA four warp groups work on up to four windows at the same time (copy in /
// two reducers over NVLink / copy out), three buffers of each kind.  At most
// 128 CTAs.
constexpr int kStagedMaxBuffers = 6;
struct StagedParams {
  int32_t rank;
  int32_t world_size;
  int32_t dtype;         // element type of the user buffers
  int32_t wire;          // element type in the pool and on the wire (== dtype, or 16-bit for fp32 buffers)
  int32_t use_multimem;  // 1: multimem.ld_reduce / multimem.st; 0: peer loads + peer stores
  int32_t use_tma;       // 1: the local copies are bulk asynchronous copies (needs wire == dtype)
  PeerTable peers;
  const void* sendbuf;   // 16-byte aligned
  void* recvbuf;         // 16-byte aligned
  uint64_t len_elements; // a whole number of 16-byte wire vectors
  double scale;
  uint64_t window_elems; // elements per window (a whole number of vectors per rank and CTA)
  // The staging memory as every rank maps it (the arena, or a larger block
  // the communicator allocated for large messages) and its multicast alias.
  unsigned char* stage[kMaxRanks];
  unsigned char* mc_stage;
  uint64_t in_off[kStagedMaxBuffers];    // byte offsets of the input windows inside the staging memory
  uint64_t out_off[kStagedMaxBuffers];   // ... and of the output windows
  int32_t buffers;       // windows of each kind in use (3 .. kStagedMaxBuffers)
  int32_t split_ctas;    // 1: the grid is 2 n blocks, [0, n) reduce and [n, 2n) copy; 0: every block does both
  uint64_t timeout_ns;
  DeviceStatus* status;
  uint32_t* doorbell;
  DeviceTraceRec* trace;   // [CTA][trace_capacity]: per window, when the reduce could start and when it was done
  int32_t trace_capacity;  // 0 = tracing off
  // W > 0: the other roles stamp too, W = number of windows, 4 W <= trace_capacity.  Records [W, 2W): the
  // loader (input buffer free, input window published), [2W, 3W): the storer (window reduced everywhere,
  // output buffer released), [3W, 4W): t_wait_done = the reducers' last store issued (before the fence).
  int32_t trace_roles;
  // Split mode: groups per role (1 .. 4) that take the windows in turn.  groups x reducing blocks <= 256
  // (a group has flag rows of its own).
  int32_t load_groups, reduce_groups, store_groups;
  int32_t posters;  // split mode: a poster warp per reducer group fences and publishes behind the data warps
};
cudaError_t LaunchStagedKernel(const StagedParams& p, const StagedParams* emu, int emu_ranks, int blocks, cudaStream_t stream);
// Largest grid of the staged kernel that is co-resident on `device` (0 on error).
int StagedKernelMaxCoResidentBlocks(int device);

// ---- reduce-scatter / all-gather (the halves of the two-shot allreduce) ----
enum RsAgMode : int32_t { kRsAgReduceScatter = 1, kRsAgAllGather = 2 };
struct RsAgParams {
  int32_t rank;
  int32_t world_size;
  int32_t dtype;
  int32_t use_multimem;  // 1: multimem.ld_reduce / multimem.st; 0: peer loads / peer stores
  int32_t mode;          // RsAgMode
  int32_t staged;        // the remote side is the pool (window by window), not a mapped user buffer
  PeerTable peers;
  const void* sendbuf;   // reduce-scatter: ws blocks; all-gather: one block
  void* recvbuf;         // reduce-scatter: one block; all-gather: ws blocks
  uint64_t block_elems;  // elements per block (per rank)
  double scale;          // reduce-scatter only
  // The remote side as every rank sees it (reduce-scatter: the inputs,
  // all-gather: the outputs): user buffers or pool windows, and their
  // multicast alias (null without multimem).
  unsigned char* peer_buf[kMaxRanks];
  unsigned char* mc_buf;
  // Block elements per window (the whole block when not staged) and the
  // distance in bytes between two sub-blocks of the remote side.
  uint64_t window_elems;
  uint64_t sub_stride_bytes;
  uint64_t timeout_ns;
  DeviceStatus* status;
  uint32_t* doorbell;
};
cudaError_t LaunchRsAgKernel(const RsAgParams& p, const RsAgParams* emu, int emu_ranks, int blocks, cudaStream_t stream);

// ---- one-shot allreduce for small messages (push to every peer, sum locally) ----
struct OneShotParams {
  int32_t rank;
  int32_t world_size;
  int32_t dtype;
  int32_t pad_;
  PeerTable peers;
  const void* sendbuf;
  void* recvbuf;
  uint64_t len_elements;
  double scale;
  uint64_t slot_offset;   // byte offset of the one-shot area in the arena
  uint64_t slot_bytes;    // bytes reserved per (parity, source rank)
  uint64_t timeout_ns;
  DeviceStatus* status;
  uint32_t* doorbell;
};
cudaError_t LaunchOneShotKernel(const OneShotParams& p, const OneShotParams* emu, int emu_ranks, int blocks, cudaStream_t stream);

// ---- two-sided device messaging through the peer's mailbox ----
struct P2pParams {
  int32_t rank;
  int32_t peer;
  int32_t is_send;
  int32_t world_size;
  PeerTable peers;
  const void* src;        // send: user buffer
  void* dst;              // recv: user buffer
  uint64_t bytes;
  uint64_t mailbox_offset;  // byte offset of the mailbox area in the arena
  uint64_t slot_bytes;      // bytes per mailbox slot
  uint32_t slots;           // slots per source rank
  uint32_t pad_;
  uint64_t first_piece;     // cumulative piece counter of this pair at call start
  uint64_t seq;
  uint64_t timeout_ns;
  DeviceStatus* status;
  uint32_t* doorbell;
};
// `ctas` (1..kP2pCtas) must be the same for every message of a communicator
// and on both sides: a CTA's flags count the pieces of its own part.  One SM
// sustains roughly 10 GB/s of stores to a peer, so bandwidth needs many CTAs.
cudaError_t LaunchP2pKernel(const P2pParams& p, int ctas, cudaStream_t stream);

// ---- device broadcast through NVSwitch multicast ----
// The root writes every piece ONCE (`multimem.st` into the broadcast ring of
// all ranks' mailbox areas at the same time, then the flag the same way); the
// others copy it out and return credits.  Needs the multicast alias of the
// arenas and a length that is a multiple of 16 (conditions every rank decides
// alike; a buffer that is only byte-aligned is moved byte by byte).
struct BcastParams {
  int32_t rank;
  int32_t root;
  int32_t world_size;
  int32_t pad_;
  PeerTable peers;
  void* buf;                // root: source, others: destination
  uint64_t bytes;
  uint64_t ring_offset;     // byte offset of the broadcast ring in the arena
  uint64_t slot_bytes;
  uint32_t slots;
  uint32_t pad2_;
  uint64_t first_piece;     // cumulative piece number of the communicator's broadcasts at call start
  uint64_t seq;
  uint64_t timeout_ns;
  DeviceStatus* status;
  uint32_t* doorbell;
};
cudaError_t LaunchBcastKernel(const BcastParams& p, int ctas, cudaStream_t stream);

}  // namespace ibcomm
