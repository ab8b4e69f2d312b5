#include "engine.h"

#include <algorithm>
#include <cstdio>
#include <cstring>

#include "ibcomm/tunables.h"

namespace ibcomm {

static uint64_t AlignUp(uint64_t v, uint64_t a) { return (v + a - 1) / a * a; }

ArenaLayout MakeArenaLayout(size_t pool_bytes, size_t work_bytes, int world_size) {
  ArenaLayout l;
  uint64_t off = 0;
  l.control_offset = off;
  off += AlignUp(sizeof(ControlPage), 65536);
  l.oneshot_offset = off;
  // A one-shot call pushes the whole message to every peer, so it needs one
  // slot per (parity, source rank): few ranks get large slots.
  const uint64_t ws = static_cast<uint64_t>(world_size < 2 ? 2 : (world_size > kMaxRanks ? kMaxRanks : world_size));
  l.oneshot_slot_bytes = kOneShotAreaBytes / (2 * ws) / 4096 * 4096;
  off += kOneShotAreaBytes;
  l.mailbox_offset = off;
  // Device Send/Recv mailboxes: per source rank a ring of slots.  A slot is
  // the unit of hand-over: before a piece's flag may be raised the sending
  // CTA waits until its stores are acknowledged over NVLink (about 6 us under
  // load, measured on B200), so a piece has to be worth several microseconds
  // of link time: 4 MiB slots, four of them (two in flight from the sender's
  // two warp groups, two being emptied by the receiver).  Knobs for experiments: IBCOMM_P2P_SLOT_KIB,
  // IBCOMM_P2P_SLOTS; all ranks must agree.
  {
    int kib = Tunable("IBCOMM_P2P_SLOT_KIB", 4096);
    if (kib < 16 || kib > (64 << 10)) kib = 4096;
    int slots = Tunable("IBCOMM_P2P_SLOTS", 4);
    if (slots < 2 || slots > kP2pMaxSlots) slots = 4;
    l.mailbox_slot_bytes = static_cast<uint64_t>(kib) << 10;
    l.mailbox_slots = static_cast<uint32_t>(slots);
  }
  // One ring per source rank, plus the ring device broadcasts are multicast into.
  l.bcast_ring_offset = off + static_cast<uint64_t>(kMaxRanks) * l.mailbox_slots * l.mailbox_slot_bytes;
  off += static_cast<uint64_t>(kMaxRanks + 1) * l.mailbox_slots * l.mailbox_slot_bytes;
  l.pool_offset = off;
  l.pool_bytes = AlignUp(pool_bytes < 4096 ? 4096 : pool_bytes, 4096);
  off += l.pool_bytes;
  l.work_offset = off;
  l.work_bytes = AlignUp(work_bytes < 4096 ? 4096 : work_bytes, 4096);
  off += l.work_bytes;
  l.total_bytes = AlignUp(off, 2u << 20);
  return l;
}

// ------------------------------------------------------------- status block
void StatusBlock::Create() {
  CUDACHECK(cudaMalloc(&d_status, sizeof(DeviceStatus)));
  CUDACHECK(cudaMemset(d_status, 0, sizeof(DeviceStatus)));
  CUDACHECK(cudaHostAlloc(reinterpret_cast<void**>(&h_doorbell), 64, cudaHostAllocMapped | cudaHostAllocPortable));
  *h_doorbell = 0;
  CUDACHECK(cudaHostGetDevicePointer(reinterpret_cast<void**>(&d_doorbell), h_doorbell, 0));
}

void StatusBlock::Destroy() {
  if (d_status != nullptr) cudaFree(d_status);
  if (h_doorbell != nullptr) cudaFreeHost(h_doorbell);
  d_status = nullptr;
  h_doorbell = nullptr;
  d_doorbell = nullptr;
  (void)cudaGetLastError();
}

uint32_t StatusBlock::Consume(DeviceStatus* out, cudaStream_t stream) {
  if (h_doorbell == nullptr) return 0;
  uint32_t bell = *reinterpret_cast<volatile uint32_t*>(h_doorbell);
  if (bell == 0) return 0;
  DeviceStatus st;
  memset(&st, 0, sizeof(st));
  CUDACHECK(cudaMemcpyAsync(&st, d_status, sizeof(st), cudaMemcpyDeviceToHost, stream));
  CUDACHECK(cudaMemsetAsync(d_status, 0, sizeof(st), stream));
  CUDACHECK(cudaStreamSynchronize(stream));
  *reinterpret_cast<volatile uint32_t*>(h_doorbell) = 0;
  if (st.code == 0) st.code = bell;
  if (out != nullptr) *out = st;
  return st.code;
}

std::string DescribeStatus(const DeviceStatus& st) {
  static const char* const codes[] = {"ok", "wait timed out", "aborted by a peer", "bad program", "message length mismatch"};
  static const char* const kinds[] = {"?", "barrier", "data flag", "slot credit", "mailbox", "one-shot flag"};
  char buf[320];
  snprintf(buf, sizeof(buf),
           "device collective failed: %s while waiting for a %s from rank %d (rank %d, channel %d, op %d, call %llu, "
           "expected %llu, saw %llu)",
           codes[st.code < 5 ? st.code : 0], kinds[st.kind < 6 ? st.kind : 0], st.peer, st.rank, st.channel, st.op_index,
           static_cast<unsigned long long>(st.seq), static_cast<unsigned long long>(st.expected & 0xffffffffull),
           static_cast<unsigned long long>(st.seen & 0xffffffffull));
  return buf;
}

// ------------------------------------------------------------ program cache
ProgramCache::~ProgramCache() { Clear(); }

void ProgramCache::Clear() {
  cache_.clear();
  for (Slab& sl : slabs_) {
    if (sl.d != nullptr) cudaFree(sl.d);
    if (sl.h != nullptr) cudaFreeHost(sl.h);
  }
  slabs_.clear();
  (void)cudaGetLastError();
}

Op* ProgramCache::Place(const std::vector<Op>& ops, cudaStream_t stream, int* slab_index) {
  const size_t n = ops.size();
  int at = -1;
  for (size_t i = 0; i < slabs_.size(); ++i)
    if (slabs_[i].cap - slabs_[i].used >= n) at = static_cast<int>(i);
  if (at < 0) {
    Slab sl;
    sl.cap = std::max<size_t>(n, (1u << 20) / sizeof(Op));
    CUDACHECK(cudaMalloc(&sl.d, sl.cap * sizeof(Op)));
    CUDACHECK(cudaHostAlloc(reinterpret_cast<void**>(&sl.h), sl.cap * sizeof(Op), cudaHostAllocPortable));
    slabs_.push_back(sl);
    at = static_cast<int>(slabs_.size()) - 1;
  }
  Slab& sl = slabs_[static_cast<size_t>(at)];
  memcpy(sl.h + sl.used, ops.data(), n * sizeof(Op));
  CUDACHECK(cudaMemcpyAsync(sl.d + sl.used, sl.h + sl.used, n * sizeof(Op), cudaMemcpyHostToDevice, stream));
  Op* d = sl.d + sl.used;
  sl.used += n;
  *slab_index = at;
  return d;
}

void ProgramCache::NoteSynchronized() {
  if (cache_.size() <= bound_) return;
  for (auto it = cache_.begin(); it != cache_.end();) {
    if (it->second->pinned) ++it;
    else it = cache_.erase(it);
  }
  // A slab without pinned programs starts over; the others keep their contents.
  for (Slab& sl : slabs_)
    if (sl.pinned == 0) sl.used = 0;
}

const CachedProgram& ProgramCache::Get(Algo algo, int rank, int world_size, size_t len_elements, DType dtype, DType wire,
                                       const ArenaLayout& layout, bool apply_scale, cudaStream_t stream, bool capturing) {
  const size_t esize = DTypeSize(dtype), wsize = DTypeSize(wire);
  // Read at the point of use, like the reference: a bad value fails the call.
  const long long env_chunk = env::ReadChunkSize();
  const bool ring = algo == Algo::kRing;
  // The ring stages in the pool.  Rabenseifner lands its pieces in the work
  // region and, since one collective runs at a time, in the pool in front of
  // it as well (the two are adjacent in the arena).
  const uint64_t stage_off = layout.pool_offset;
  const uint64_t stage_bytes = ring ? layout.pool_bytes : layout.pool_bytes + layout.work_bytes;
  // Knobs that shape the program are part of the key: the ring's chunks per
  // rank and the number of pieces Rabenseifner cuts the message into.
  const size_t ring_cpr = ring ? RingChunksPerRank(len_elements, esize, static_cast<size_t>(world_size)) : 0;
  int raben_div = Tunable("IBCOMM_RABEN_PIECES", 8);
  if (raben_div < 1 || raben_div > 1024) raben_div = 8;
  Key key{static_cast<int>(algo), rank, world_size, len_elements, static_cast<int>(dtype), static_cast<int>(wire),
          env_chunk, apply_scale, stage_off, stage_bytes, ring ? static_cast<int>(ring_cpr) : raben_div};
  auto it = cache_.find(key);
  if (it != cache_.end()) {
    CachedProgram& hit = *it->second;
    if (capturing && !hit.pinned) {
      hit.pinned = true;
      if (hit.slab >= 0) ++slabs_[static_cast<size_t>(hit.slab)].pinned;
    }
    return hit;
  }

  const int regions = NumRegions(algo, world_size);
  ProgramRequest req;
  req.algo = algo;
  req.rank = rank;
  req.world_size = world_size;
  if (ring) {
    // At least four slots keep the pipeline moving; two is the minimum the
    // schedule needs.
    uint64_t max_chunk_wire = stage_bytes / (static_cast<uint64_t>(regions) * 4) / 128 * 128;
    if (max_chunk_wire < 128) max_chunk_wire = 128;
    const size_t max_chunk_user = static_cast<size_t>(max_chunk_wire / wsize * esize);
    req.ranges = SplitForDevice(len_elements, esize, static_cast<size_t>(world_size), env_chunk, max_chunk_user, ring_cpr);
  } else {
    // Chunks only fix the block boundaries here; what travels are pieces:
    // IBCOMM_CHUNKSIZE when set, otherwise an eighth of the message (four
    // pieces in the largest step; knob IBCOMM_RABEN_PIECES), as far as two
    // slots per partner fit.
    req.ranges = SplitForDevice(len_elements, esize, static_cast<size_t>(world_size), env_chunk, 0);
    size_t cap = static_cast<size_t>(stage_bytes / (static_cast<uint64_t>(regions) * 2) / wsize) / 32 * 32;
    if (cap < 32) cap = 32;
    size_t piece = env_chunk > 0 ? static_cast<size_t>(env_chunk) / esize : std::max<size_t>(util::ceilDiv(len_elements, static_cast<size_t>(raben_div)), 16384);
    if (piece > cap) {
      static bool warned = false;
      if (!warned && rank == 0) {
        warned = true;
        IBCOMM_WARN("IBCOMM_MEMORY_POOL_PRE_ALLOC + IBCOMM_WORK_GPU_MEMORY_SIZE (%llu bytes) limit Rabenseifner's transfer "
                    "pieces to %zu bytes instead of %zu; increase them for large messages.\n",
                    static_cast<unsigned long long>(stage_bytes), cap * wsize, piece * wsize);
      }
      piece = cap;
    }
    if (env_chunk <= 0 && piece >= 32) piece = util::ceilDiv(piece, size_t(32)) * 32;
    req.piece_elems = piece;
  }
  req.wire_elem_bytes = wsize;
  req.stage_offset = stage_off;
  req.stage_bytes = stage_bytes;
  req.apply_scale = apply_scale;
  std::unique_ptr<CachedProgram> cp(new CachedProgram());
  cp->prog = BuildProgram(req);
  {
    const std::string bad = ValidateProgram(cp->prog, len_elements, wsize, world_size);
    if (!bad.empty()) IBCOMM_FAIL(INVALID_ARGUMENT, "Internal error: the %s program for %zu elements on %d ranks is out of bounds (%s).\n",
                                  ring ? "ring" : "Rabenseifner", len_elements, world_size, bad.c_str());
  }
  if (!cp->prog.ops.empty()) {
    cp->d_ops = Place(cp->prog.ops, stream, &cp->slab);
    if (capturing) {
      cp->pinned = true;
      ++slabs_[static_cast<size_t>(cp->slab)].pinned;
    }
  }
  const CachedProgram& ref = *cp;
  cache_[key] = std::move(cp);
  return ref;
}

ExecParams MakeExecParams(const RankResources& rr, const CachedProgram& cp, DType dtype, DType wire, const void* sendbuf,
                          void* recvbuf, size_t len_elements, double scale, uint64_t timeout_ns,
                          DeviceTraceRec* trace, int trace_capacity) {
  ExecParams p;
  memset(&p, 0, sizeof(p));
  p.rank = rr.rank;
  p.world_size = rr.world_size;
  p.dtype = static_cast<int32_t>(dtype);
  p.wire = static_cast<int32_t>(wire);
  p.peers = rr.peers;
  p.sendbuf = sendbuf;
  p.recvbuf = recvbuf;
  p.len_elements = len_elements;
  p.scale = scale;
  p.ops = cp.d_ops;
  p.num_ops = static_cast<int32_t>(cp.prog.ops.size());
  p.trace_capacity = trace_capacity;
  p.stage = cp.prog.stage;
  p.timeout_ns = timeout_ns;
  p.status = rr.d_status;
  p.doorbell = rr.d_doorbell;
  p.trace = trace;
  return p;
}

OneShotParams MakeOneShotParams(const RankResources& rr, DType dtype, const void* sendbuf, void* recvbuf,
                                size_t len_elements, double scale, uint64_t timeout_ns) {
  OneShotParams p;
  memset(&p, 0, sizeof(p));
  p.rank = rr.rank;
  p.world_size = rr.world_size;
  p.dtype = static_cast<int32_t>(dtype);
  p.peers = rr.peers;
  p.sendbuf = sendbuf;
  p.recvbuf = recvbuf;
  p.len_elements = len_elements;
  p.scale = scale;
  p.slot_offset = rr.layout.oneshot_offset;
  p.slot_bytes = rr.layout.oneshot_slot_bytes;
  p.timeout_ns = timeout_ns;
  p.status = rr.d_status;
  p.doorbell = rr.d_doorbell;
  return p;
}

}  // namespace ibcomm
