// Plain structs shared by the host runtime and the sm_100a kernels.
//
// Device collectives run as ONE kernel per rank.  The point-to-point
// algorithms (ring, Rabenseifner) are expressed as a small per-rank program of
// `Op`s that the host compiles once per (algorithm, length, world size) and a
// generic kernel interprets; every op is a fused
//   wait-for-peer -> load (+ add) (+ scale) (+ cast) -> store local / store to
//   the peer's staging slot over NVLink -> post flag / return credit
// step.  This replaces the reference's per-chunk host loop of
// cudaMemcpyAsync + reduce kernel + cudaMemcpyAsync + ibv_post_send
// (ibcomm/allreduce_cuda_impl.h:103-299, 470-707).
#pragma once

#include <cstddef>
#include <cstdint>

#ifdef __CUDACC__
#define IBCOMM_HD __host__ __device__
#else
#define IBCOMM_HD
#endif

namespace ibcomm {

constexpr int kMaxRanks = 8;       // one NVSwitch box
constexpr int kMaxChannels = 256;  // CTAs per rank a collective may use
constexpr int kExecThreads = 512;  // threads per channel CTA
constexpr int kP2pCtas = 128;      // most CTAs a device Send / Recv / Bcast kernel may use (each owns a fixed part of every mailbox slot)
constexpr int kP2pMaxSlots = 8;    // upper bound of mailbox slots per source rank

// ---- control page at the start of every rank's arena (peer-writable) ----
// All words are 64-bit, written by exactly one remote rank and polled locally.
// Values only grow: (call sequence << 32) | count.
struct ControlPage {
  // bar[c][s]: rank s announces "my channel c reached barrier point v".
  uint64_t bar[kMaxChannels][kMaxRanks];
  // inflag[c][s]: number of transfers rank s has completed into my staging.
  uint64_t inflag[kMaxChannels][kMaxRanks];
  // credit[c][d]: number of my transfers rank d has consumed.
  uint64_t credit[kMaxChannels][kMaxRanks];
  // Point-to-point mailbox counters per CTA of the Send / Recv kernels and
  // per source / destination rank: cumulative piece numbers of the ordered
  // pair.  p2p_len[s][slot]: byte length of the message from rank s whose
  // first piece sits in `slot` (written before that piece's flag).
  uint64_t p2p_flag[kP2pCtas][kMaxRanks];
  uint64_t p2p_credit[kP2pCtas][kMaxRanks];
  uint64_t p2p_len[kMaxRanks][kP2pMaxSlots];
  // Device broadcast through the switch: the root multicasts pieces into the
  // broadcast ring of every rank's mailbox area and then bcast_flag (the
  // cumulative piece number over all broadcasts of the communicator);
  // receiver q returns bcast_credit[c][q] to every rank, so that whoever is
  // the root of a later broadcast knows which slots are free.
  uint64_t bcast_flag[kP2pCtas];
  uint64_t bcast_credit[kP2pCtas][kMaxRanks];
  // Set (to the call sequence) by any rank that gave up; polled by waiters.
  uint64_t abort_seq;
  // Written only by this rank's own kernels: the number of collectives it has
  // completed, and how many CTAs of the running one have finished.  Every
  // collective kernel takes its sequence number from here (call_seq + 1) and
  // the last CTA to finish publishes it, so a kernel's parameters carry
  // nothing that changes from call to call and a captured CUDA graph of
  // collectives can be replayed.  All ranks issue the same collectives in the
  // same order, so their counters agree.
  uint64_t call_seq;
  uint32_t done_ctas;
  uint32_t pad32_;
  uint64_t pad_[5];
  // One-shot allreduce flags: [parity][cta][source].
  uint64_t oneshot_flag[2][kMaxChannels][kMaxRanks];
};

// ---- error report written by a kernel whose bounded wait ran out ----
enum DeviceStatusCode : uint32_t {
  kStatusOk = 0,
  kStatusWaitTimeout = 1,   // a flag did not arrive within the limit
  kStatusPeerAbort = 2,     // a peer (or another CTA) reported failure
  kStatusBadProgram = 3,    // self-check of an op failed (index out of range)
  kStatusLengthMismatch = 4,  // a device Recv met a message of another length than it was posted for
};
enum DeviceWaitKind : uint32_t { kWaitBarrier = 1, kWaitData = 2, kWaitCredit = 3, kWaitP2p = 4, kWaitOneShot = 5 };

struct DeviceStatus {
  uint32_t code;      // DeviceStatusCode; first failure wins
  uint32_t kind;      // DeviceWaitKind
  int32_t rank;
  int32_t peer;
  int32_t channel;
  int32_t op_index;
  uint64_t expected;
  uint64_t seen;
  uint64_t seq;
};

// ---- per-step trace record (optional) ----
struct DeviceTraceRec {
  uint64_t t_wait_done;  // %globaltimer when the op's waits were satisfied
  uint64_t t_done;       // %globaltimer when the op's flags were posted
};

// ---- program ops ----
enum OpSrc : uint8_t { kSrcNone = 0, kSrcSend = 1, kSrcRecv = 2, kSrcStage = 3 };
enum OpFlags : uint8_t {
  kOpScale = 1,        // multiply by ExecParams::scale before storing
  kOpStoreLocal = 2,   // store to recvbuf[range]
  kOpStoreRemote = 4,  // store to peer_out's staging slot
  // The value is final: round it through the wire type before the local store,
  // so that the owner keeps the same bits every other rank will receive.
  kOpRoundWire = 8,
};

struct Op {
  uint8_t src_a;     // OpSrc
  uint8_t src_b;     // OpSrc (added to src_a); kSrcNone = plain copy
  uint8_t flags;     // OpFlags
  int8_t peer_in;    // rank whose transfer feeds kSrcStage, -1 if none
  int8_t peer_out;   // rank that receives the remote store, -1 if none
  uint8_t region_in;   // staging region index on my side (one per in-peer)
  uint8_t region_out;  // staging region index on peer_out's side
  uint8_t pad_;
  uint32_t slot_in;    // staging slot index inside region_in
  uint32_t slot_out;   // staging slot index inside region_out
  uint32_t wait_in;      // wait until inflag[ch][peer_in] >= base + wait_in   (0 = no wait)
  uint32_t wait_credit;  // wait until credit[ch][peer_out] >= base + wait_credit (0 = no wait)
  uint32_t post_out;     // then peer_out.inflag[ch][me] = base + post_out     (0 = no post)
  uint32_t post_credit;  // and  peer_in.credit[ch][me] = base + post_credit   (0 = no post)
  uint64_t elem_begin;   // range in elements of the message
  uint64_t elem_count;
  // First element of the slot-sized cell the range lies in (<= elem_begin).
  // Staging offsets and the split among channels are relative to the cell, so
  // an element keeps its channel and its place in a slot in every op.
  uint64_t cell_begin;
};

// Geometry of the staging area a program runs in.
struct StageLayout {
  uint64_t offset;       // byte offset of the area inside the arena
  uint64_t slot_bytes;   // bytes of one slot (multiple of 128)
  uint32_t slots;        // slots per region
  uint32_t regions;      // number of regions (= distinct in-peers)
};

// Cell-relative elements [*lo, *hi) that channel `c` of `nch` handles of an op
// that covers [first, first + count) of its cell.  The cut depends only on the
// slot capacity (`slot_elems`), never on the op: a staging slot is reused by
// ranges of different lengths, and the credit a channel receives covers
// exactly the byte range that channel owns in every slot; likewise an element
// is always handled by the same channel, whatever range an op names.  Slices
// start on multiples of kSliceAlign elements, so a slice is 16-byte aligned in
// every element type whenever its cell is.
constexpr uint32_t kSliceAlign = 64;
IBCOMM_HD inline void ChannelSlice(uint64_t first, uint64_t count, uint64_t slot_elems, int nch, int c, uint64_t* lo,
                                   uint64_t* hi) {
  if (slot_elems < first + count) slot_elems = first + count;
  uint64_t per = (slot_elems + static_cast<uint64_t>(nch) - 1) / static_cast<uint64_t>(nch);
  per = (per + kSliceAlign - 1) / kSliceAlign * kSliceAlign;
  uint64_t b = per * static_cast<uint64_t>(c);
  uint64_t e = b + per;
  if (b < first) b = first;
  if (e > first + count) e = first + count;
  if (b > e) b = e;
  *lo = b;
  *hi = e;
}

// ---- how the two-shot kernels split a staging window among ranks and CTAs ----
// [*b, *e) = part `part` of `parts` of the range [lo, hi).
IBCOMM_HD inline void SubRange(uint64_t lo, uint64_t hi, int part, int parts, uint64_t* b, uint64_t* e) {
  const uint64_t len = hi - lo;
  const uint64_t per = (len + static_cast<uint64_t>(parts) - 1) / static_cast<uint64_t>(parts);
  uint64_t x = lo + per * static_cast<uint64_t>(part);
  if (x > hi) x = hi;
  uint64_t y = x + per;
  if (y > hi) y = hi;
  *b = x;
  *e = y;
}

// Part `part` of `parts` of shard `s` of a window, in 16-byte vectors.  The
// split is that of a FULL window (`full_nvec` vectors) clipped to the `nvec`
// vectors this window holds: a CTA then covers the same bytes of the staging
// windows in every window of a call, the short last one included.  The
// barriers are per CTA, so they order a CTA's accesses only against the same
// CTA of the other ranks; a split that moved with the window's length would
// let a CTA that is one window ahead overwrite bytes that another CTA has not
// copied out yet.
IBCOMM_HD inline void WindowPart(uint64_t full_nvec, uint64_t nvec, int s, int ws, int part, int parts, uint64_t* b,
                                           uint64_t* e) {
  uint64_t sb, se;
  SubRange(0, full_nvec, s, ws, &sb, &se);
  SubRange(sb, se, part, parts, b, e);
  if (*b > nvec) *b = nvec;
  if (*e > nvec) *e = nvec;
}

struct PeerTable {
  unsigned char* arena[kMaxRanks];  // every rank's arena as mapped here
  unsigned char* mc_arena;          // multicast alias of the arenas, or null
};

struct ExecParams {
  int32_t rank;
  int32_t world_size;
  int32_t dtype;       // DType of the user buffers
  int32_t wire;        // DType on the wire / in staging
  PeerTable peers;
  const void* sendbuf;
  void* recvbuf;
  uint64_t len_elements;
  double scale;
  const Op* ops;
  int32_t num_ops;
  int32_t trace_capacity;  // records per channel, 0 = tracing off
  StageLayout stage;
  uint64_t timeout_ns;   // limit of every wait
  DeviceStatus* status;  // device memory, fetched by the host after a failure
  uint32_t* doorbell;    // host-mapped word a failing kernel sets non-zero
  DeviceTraceRec* trace; // [channel][trace_capacity]
};

}  // namespace ibcomm
