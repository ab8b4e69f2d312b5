// Schedule compiler: turns (algorithm, rank, world size, chunk ranges) into the
// per-rank op program the device executor interprets (see device_types.h).
//
// Ring (reference ibcomm/allreduce_cuda_impl.h:35-301): reduce-scatter then
// all-gather around the ring r-1 -> r -> r+1, chunk-pipelined; after the
// reduce-scatter rank r owns the reduced block of rank r+1, and inside a
// block chunk ids descend.  The wire order is position-major (the i-th chunk
// of every block travels before the (i+1)-th of any), which keeps the
// schedule deadlock-free with as few as two staging slots.
//
// Rabenseifner (reference :326-717): recursive halving with the partner
// rank ^ (1 << s), nearest first, the lower rank giving away the front part;
// recursive doubling in mirror order; every rank-block moves as its pipeline
// chunks.  World sizes that are not a power of two are folded first: ranks
// below 2 * (ws - 2^k) pair up, swap halves and add, the even rank hands its
// half over and sits out, and gets the result back at the end.
#pragma once

#include <string>
#include <vector>

#include "ibcomm/communicator.h"
#include "ibcomm/device_types.h"

namespace ibcomm {

struct ProgramRequest {
  Algo algo = Algo::kRing;
  int rank = 0;
  int world_size = 1;
  std::vector<Range> ranges;      // pipeline chunks of the message, in elements
  // Rabenseifner only: length of a transfer piece in elements.  0 = one piece
  // per chunk.  A step moves a contiguous run of chunks, so with a piece
  // length the run is cut into pieces of that length regardless of chunk
  // boundaries (fewer, larger ops).  Must be the same on every rank.
  size_t piece_elems = 0;
  size_t wire_elem_bytes = 4;     // element size in staging
  uint64_t stage_offset = 0;      // where the staging area starts in the arena
  uint64_t stage_bytes = 0;       // how large it is
  bool apply_scale = false;
};

struct Program {
  std::vector<Op> ops;
  StageLayout stage{};
  std::vector<int> in_peers;  // region index -> source rank, for this rank
  // Transfers per peer over the whole program, for tests and credit audits.
  uint32_t sent_to[kMaxRanks] = {0};
  uint32_t received_from[kMaxRanks] = {0};
};

// Ordered list of the ranks that store into `rank`'s staging area.  The index
// in this list is the staging region the sender must address.
std::vector<int> InPeers(Algo algo, int rank, int world_size);
// Regions every rank reserves (the maximum of InPeers over ranks).
int NumRegions(Algo algo, int world_size);

// Largest chunk, in elements.
size_t MaxChunkElems(const std::vector<Range>& ranges);
// Staging geometry for a request; slots == 0 means the area is too small for
// two slots per region and the caller has to cut smaller chunks.
StageLayout PlanStage(const ProgramRequest& req);

Program BuildProgram(const ProgramRequest& req);

// Chunk cut used by the device paths: the reference's rules and exit codes
// (SplitBuffer), but when IBCOMM_CHUNKSIZE is unset the chunk length is
// rounded up to a multiple of 128 bytes so that every chunk starts on a
// vector boundary, and chunks are cut again (each into the same number of
// pieces, which keeps block boundaries) until one fits `max_chunk_bytes`.
// `chunks_per_rank` replaces the reference's 4 (chunks = 4 * world_size) when
// IBCOMM_CHUNKSIZE is unset: small messages are cut into fewer chunks, so
// that a ring step moves a useful amount of data (see RingChunksPerRank).
std::vector<Range> SplitForDevice(size_t len_elements, size_t elem_bytes, size_t world_size,
                                  int64_t env_chunk_bytes, size_t max_chunk_bytes, size_t chunks_per_rank = 4);
// Chunks per rank of the device ring when IBCOMM_CHUNKSIZE is unset: the
// reference's 4 (knob IBCOMM_RING_POSITIONS) as long as a chunk then holds at
// least IBCOMM_RING_MIN_CHUNK bytes (default 16 KiB), fewer (down to one)
// below that: a 4 KiB message on 8 ranks is one 512-byte chunk per rank and
// 15 ring steps instead of 32 chunks and 60 steps.
size_t RingChunksPerRank(size_t len_elements, size_t elem_bytes, size_t world_size);

std::string DescribeOp(const Op& op);

// Elements per staging window of the two-shot kernel for a message of `n`
// elements when a window can hold `cap_elems`: as few windows as fit, of equal
// size (the kernel splits every window as a full one, so a much shorter last
// window would leave most of its CTAs idle), a whole number of 16-byte
// vectors per rank and channel.
uint64_t TwoShotWindowElems(uint64_t n, uint64_t cap_elems, size_t esize, int world_size, int channels);

// Bounds check of a program before it is handed to the device: every op's
// message range inside `len_elements`, its place inside a staging slot, and
// its slot, region and peer indices inside the program's stage geometry.
// Returns an empty string, or a description of the first offending op.  The
// executor kernel repeats the check per op and reports "bad program" instead
// of touching memory.
std::string ValidateProgram(const Program& prog, uint64_t len_elements, size_t wire_elem_bytes, int world_size);

}  // namespace ibcomm
