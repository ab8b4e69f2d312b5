#include "ibcomm/schedule.h"

#include <algorithm>
#include <cstdio>

#include "ibcomm/tunables.h"

namespace ibcomm {

namespace {

inline int Mod(int x, int m) { return ((x % m) + m) % m; }

// Per-rank program under construction with the per-peer transfer counters
// that make both ends of a pair agree on slot numbers and flag values.
struct Builder {
  const ProgramRequest& req;
  Program prog;
  uint32_t slots;
  std::vector<int> my_in_peers;

  explicit Builder(const ProgramRequest& r) : req(r) {
    prog.stage = PlanStage(r);
    slots = prog.stage.slots;
    my_in_peers = InPeers(r.algo, r.rank, r.world_size);
    prog.in_peers = my_in_peers;
  }

  int RegionOf(int receiver, int sender) const {
    std::vector<int> peers = (receiver == req.rank) ? my_in_peers : InPeers(req.algo, receiver, req.world_size);
    for (size_t i = 0; i < peers.size(); ++i)
      if (peers[i] == sender) return static_cast<int>(i);
    IBCOMM_FAIL(INVALID_ARGUMENT, "schedule: rank %d is not an in-peer of rank %d.\n", sender, receiver);
  }

  Op Base(const Range& g) const {
    Op op{};
    op.peer_in = -1;
    op.peer_out = -1;
    op.elem_begin = g.first;
    op.elem_count = g.second - g.first;
    op.cell_begin = g.first;
    if (req.algo == Algo::kRabenseifner && req.piece_elems != 0) op.cell_begin = g.first / req.piece_elems * req.piece_elems;
    return op;
  }
  Range ChunkRange(int chunk) const { return req.ranges[static_cast<size_t>(chunk)]; }

  // Cuts the contiguous chunk list `chunks` into transfer pieces: one piece per
  // chunk, or, when the request names a piece length, pieces of that length
  // over the whole contiguous element range (fewer, larger ops).
  std::vector<Range> Pieces(const std::vector<int>& chunks) const {
    std::vector<Range> out;
    if (chunks.empty()) return out;
    if (req.piece_elems == 0 || req.algo != Algo::kRabenseifner) {
      for (int c : chunks) out.push_back(ChunkRange(c));
      return out;
    }
    // Pieces are the cells of a fixed grid over the message (multiples of the
    // piece length), clipped to the run: an element lies in the same cell in
    // every step.
    const size_t b = ChunkRange(chunks.front()).first, e = ChunkRange(chunks.back()).second;
    size_t x = b;
    while (x < e) {
      const size_t cell_end = (x / req.piece_elems + 1) * req.piece_elems;
      out.emplace_back(x, std::min(e, cell_end));
      x = std::min(e, cell_end);
    }
    return out;
  }

  void AttachOut(Op* op, int to) {
    uint32_t k = prog.sent_to[to]++;
    op->flags |= kOpStoreRemote;
    op->peer_out = static_cast<int8_t>(to);
    op->region_out = static_cast<uint8_t>(RegionOf(to, req.rank));
    op->slot_out = k % slots;
    op->wait_credit = k >= slots ? k - slots + 1 : 0;
    op->post_out = k + 1;
  }

  void AttachIn(Op* op, int from) {
    uint32_t k = prog.received_from[from]++;
    op->peer_in = static_cast<int8_t>(from);
    op->region_in = static_cast<uint8_t>(RegionOf(req.rank, from));
    op->slot_in = k % slots;
    op->wait_in = k + 1;
    op->post_credit = k + 1;
  }

  // Plain send of a chunk taken from `src` (sendbuf or recvbuf).
  void Send(const Range& g, OpSrc src, int to) {
    Op op = Base(g);
    op.src_a = src;
    AttachOut(&op, to);
    prog.ops.push_back(op);
  }

  // Receive a chunk; optionally add `add` to it, store locally and/or forward.
  void Recv(const Range& g, int from, OpSrc add, bool store_local, bool scale, int forward_to) {
    Op op = Base(g);
    op.src_a = kSrcStage;
    op.src_b = add;
    if (store_local) op.flags |= kOpStoreLocal;
    if (scale) op.flags |= kOpRoundWire;
    if (scale && req.apply_scale) op.flags |= kOpScale;
    AttachIn(&op, from);
    if (forward_to >= 0) AttachOut(&op, forward_to);
    prog.ops.push_back(op);
  }

  // One exchange step with a single partner: `sends` leave, `recvs` arrive.
  // Sends run at most `slots` ahead of the receives so that neither side can
  // block on credits the other side has not had a chance to return.
  void Exchange(int peer, const std::vector<int>& send_chunks, OpSrc send_src, const std::vector<int>& recv_chunks,
                OpSrc recv_add, bool recv_scale) {
    const std::vector<Range> sends = Pieces(send_chunks), recvs = Pieces(recv_chunks);
    size_t si = 0, ri = 0;
    const size_t ahead = slots;
    while (si < sends.size() && si < ahead) Send(sends[si++], send_src, peer);
    while (ri < recvs.size()) {
      Recv(recvs[ri], peer, recv_add, true, recv_scale, -1);
      ++ri;
      if (si < sends.size()) Send(sends[si++], send_src, peer);
    }
    while (si < sends.size()) Send(sends[si++], send_src, peer);
  }
};

std::vector<int> ChunksOfBlocks(const std::vector<std::vector<int>>& blocks, int b, int e) {
  std::vector<int> out;
  for (int i = b; i < e; ++i) out.insert(out.end(), blocks[static_cast<size_t>(i)].begin(), blocks[static_cast<size_t>(i)].end());
  return out;
}

void BuildRing(Builder* bld) {
  const ProgramRequest& q = bld->req;
  const int ws = q.world_size, r = q.rank;
  const int from = Mod(r - 1, ws), to = Mod(r + 1, ws);
  const std::vector<std::vector<int>> blocks = GetRankToChunk(q.ranges.size(), static_cast<size_t>(ws));
  size_t positions = 0;
  for (const auto& b : blocks) positions = std::max(positions, b.size());
  // i-th chunk of a block, ids descending inside the block.
  auto at = [&](int blk, size_t i) -> int {
    const std::vector<int>& b = blocks[static_cast<size_t>(blk)];
    return i < b.size() ? b[b.size() - 1 - i] : -1;
  };
  // Chunks at the same position of their blocks form a chain: every op of a
  // chain waits for the op the upstream rank ran one step earlier.  Chains
  // are independent of each other, so a group of them is walked step by step
  // (all chains' step k before any chain's step k + 1): while one chain's
  // flag travels, the CTA moves the others' data.  A group of g chains keeps
  // up to g transfers ahead of the downstream rank's receives, so it needs
  // g + 1 staging slots (with g slots every rank would wait for a credit that
  // its neighbour can only return after the same wait).
  const size_t group = std::max<size_t>(1, std::min<size_t>(positions, bld->slots > 1 ? bld->slots - 1 : 1));
  for (size_t i0 = 0; i0 < positions; i0 += group) {
    const size_t i1 = std::min(positions, i0 + group);
    for (size_t i = i0; i < i1; ++i) {
      const int c = at(r, i);
      if (c >= 0) bld->Send(bld->ChunkRange(c), kSrcSend, to);
    }
    for (int k = 0; k <= ws - 2; ++k) {  // reduce-scatter
      const bool final_step = (k == ws - 2);
      for (size_t i = i0; i < i1; ++i) {
        const int c = at(Mod(r - 1 - k, ws), i);
        if (c < 0) continue;
        bld->Recv(bld->ChunkRange(c), from, kSrcSend, /*store_local=*/final_step, /*scale=*/final_step, to);
      }
    }
    for (int k = 0; k <= ws - 2; ++k) {  // all-gather
      for (size_t i = i0; i < i1; ++i) {
        const int c = at(Mod(r - k, ws), i);
        if (c < 0) continue;
        bld->Recv(bld->ChunkRange(c), from, kSrcNone, true, false, k != ws - 2 ? to : -1);
      }
    }
  }
}

void BuildRabenseifner(Builder* bld) {
  const ProgramRequest& q = bld->req;
  const int ws = q.world_size, r = q.rank;
  const int p = static_cast<int>(util::FloorPow2(static_cast<uint64_t>(ws)));
  const int extra = ws - p;
  const int exp = util::GetExpOfTwo(static_cast<uint64_t>(p));
  const int C = static_cast<int>(q.ranges.size());
  auto real_rank = [extra](int v) { return v < extra ? 2 * v + 1 : v + extra; };
  std::vector<int> all(static_cast<size_t>(C));
  for (int i = 0; i < C; ++i) all[static_cast<size_t>(i)] = i;
  const std::vector<int> front(all.begin(), all.begin() + C / 2), back(all.begin() + C / 2, all.end());
  const std::vector<int> none;

  int vrank;
  OpSrc partial = kSrcSend;  // where my running partial sum lives
  if (r < 2 * extra) {
    const bool even = (r & 1) == 0;
    const int partner = even ? r + 1 : r - 1;
    const std::vector<int>& keep = even ? front : back;
    const std::vector<int>& give = even ? back : front;
    bld->Exchange(partner, give, kSrcSend, keep, kSrcSend, false);
    if (even) {
      bld->Exchange(partner, keep, kSrcRecv, none, kSrcNone, false);
      vrank = -1;
    } else {
      bld->Exchange(partner, none, kSrcRecv, give, kSrcNone, false);
      vrank = r / 2;
      partial = kSrcRecv;
    }
  } else {
    vrank = r - extra;
  }

  if (vrank >= 0) {
    const std::vector<std::vector<int>> blocks = GetRankToChunk(static_cast<size_t>(C), static_cast<size_t>(p));
    int b = 0, e = p;
    for (int s = 0; s < exp; ++s) {
      const int vpeer = vrank ^ (1 << s);
      const int mid = e - (e - b) / 2;
      int sb, se, kb, ke;
      if (vrank < vpeer) {
        sb = b; se = mid; kb = mid; ke = e;
      } else {
        kb = b; ke = mid; sb = mid; se = e;
      }
      bld->Exchange(real_rank(vpeer), ChunksOfBlocks(blocks, sb, se), partial, ChunksOfBlocks(blocks, kb, ke), partial,
                    s == exp - 1);
      partial = kSrcRecv;
      b = kb;
      e = ke;
    }
    for (int s = 0; s < exp; ++s) {
      const int vpeer = vrank ^ (1 << (exp - 1 - s));
      const int w = e - b;
      int rb, re;
      if (vrank > vpeer) {
        rb = e; re = e + w;
      } else {
        rb = b - w; re = b;
      }
      bld->Exchange(real_rank(vpeer), ChunksOfBlocks(blocks, b, e), kSrcRecv, ChunksOfBlocks(blocks, rb, re), kSrcNone, false);
      b = std::min(b, rb);
      e = std::max(e, re);
    }
  }

  if (r < 2 * extra) {
    if ((r & 1) == 0) bld->Exchange(r + 1, none, kSrcRecv, all, kSrcNone, false);
    else bld->Exchange(r - 1, all, kSrcRecv, none, kSrcNone, false);
  }
}

}  // namespace

std::vector<int> InPeers(Algo algo, int rank, int world_size) {
  std::vector<int> peers;
  if (world_size <= 1) return peers;
  if (algo == Algo::kRing) {
    peers.push_back(Mod(rank - 1, world_size));
    return peers;
  }
  // Rabenseifner: fold partner first, then the halving partners by step.
  const int p = static_cast<int>(util::FloorPow2(static_cast<uint64_t>(world_size)));
  const int extra = world_size - p;
  const int exp = util::GetExpOfTwo(static_cast<uint64_t>(p));
  auto real_rank = [extra](int v) { return v < extra ? 2 * v + 1 : v + extra; };
  int vrank;
  if (rank < 2 * extra) {
    peers.push_back((rank & 1) == 0 ? rank + 1 : rank - 1);
    vrank = (rank & 1) == 0 ? -1 : rank / 2;
  } else {
    vrank = rank - extra;
  }
  if (vrank >= 0)
    for (int s = 0; s < exp; ++s) peers.push_back(real_rank(vrank ^ (1 << s)));
  return peers;
}

int NumRegions(Algo algo, int world_size) {
  int m = 1;
  for (int r = 0; r < world_size; ++r) m = std::max(m, static_cast<int>(InPeers(algo, r, world_size).size()));
  return m;
}

size_t MaxChunkElems(const std::vector<Range>& ranges) {
  size_t m = 0;
  for (const Range& g : ranges) m = std::max(m, g.second - g.first);
  return m;
}

StageLayout PlanStage(const ProgramRequest& req) {
  StageLayout st{};
  st.offset = req.stage_offset;
  st.regions = static_cast<uint32_t>(NumRegions(req.algo, req.world_size));
  // +16 so that a slice may start at the same 16-byte phase as the user data.
  const bool pieces = req.algo == Algo::kRabenseifner && req.piece_elems != 0;
  uint64_t bytes = (pieces ? req.piece_elems : MaxChunkElems(req.ranges)) * req.wire_elem_bytes;
  st.slot_bytes = (bytes + 127) & ~uint64_t(127);
  if (st.slot_bytes == 0) st.slot_bytes = 128;
  uint64_t per_region = req.stage_bytes / st.regions;
  uint64_t slots = per_region / st.slot_bytes;
  st.slots = slots > 64 ? 64u : static_cast<uint32_t>(slots);
  if (st.slots < 2) st.slots = 0;
  return st;
}

Program BuildProgram(const ProgramRequest& req) {
  if (req.world_size < 1 || req.world_size > kMaxRanks)
    IBCOMM_FAIL(NOT_SUPPORTED, "Device collectives support 1..%d ranks (got %d).\n", kMaxRanks, req.world_size);
  Builder bld(req);
  if (req.world_size == 1) return bld.prog;
  if (bld.slots == 0)
    IBCOMM_FAIL(INVALID_ARGUMENT,
                "The staging area (%llu bytes) cannot hold two slots of %llu bytes for each of %u "
                "regions.\n",
                static_cast<unsigned long long>(req.stage_bytes),
                static_cast<unsigned long long>(bld.prog.stage.slot_bytes), bld.prog.stage.regions);
  switch (req.algo) {
    case Algo::kRing: BuildRing(&bld); break;
    case Algo::kRabenseifner: BuildRabenseifner(&bld); break;
    default:
      IBCOMM_FAIL(INVALID_ARGUMENT, "No op program exists for algorithm '%s'.\n", AlgoName(req.algo));
  }
  return bld.prog;
}

std::vector<Range> SplitForDevice(size_t len_elements, size_t elem_bytes, size_t world_size,
                                  int64_t env_chunk_bytes, size_t max_chunk_bytes, size_t chunks_per_rank) {
  std::vector<Range> base = SplitBuffer(len_elements, elem_bytes, world_size, env_chunk_bytes);
  const size_t vec_elems = 128 / elem_bytes;
  if (env_chunk_bytes <= 0) {
    if (chunks_per_rank < 1) chunks_per_rank = 1;
    size_t per = util::ceilDiv(len_elements, chunks_per_rank * world_size);
    const bool round = per >= 4 * vec_elems && per % vec_elems != 0;
    if (round) per = util::ceilDiv(per, vec_elems) * vec_elems;
    if (round || chunks_per_rank != 4) {
      base.clear();
      for (size_t b = 0; b < len_elements; b += per) base.emplace_back(b, std::min(len_elements, b + per));
    }
  }
  size_t largest = MaxChunkElems(base) * elem_bytes;
  if (max_chunk_bytes == 0 || largest <= max_chunk_bytes) return base;
  // Cut every chunk into `f` pieces on 128-byte boundaries.
  const size_t f = util::ceilDiv(largest, max_chunk_bytes);
  size_t piece = util::ceilDiv(MaxChunkElems(base), f);
  piece = util::ceilDiv(piece, vec_elems) * vec_elems;
  std::vector<Range> out;
  out.reserve(base.size() * f);
  for (const Range& g : base) {
    size_t b = g.first;
    for (size_t k = 0; k < f; ++k) {
      size_t e = (k + 1 == f) ? g.second : std::min(g.second, b + piece);
      out.emplace_back(b, e);  // possibly empty; keeps f pieces per chunk
      b = e;
    }
  }
  return out;
}

size_t RingChunksPerRank(size_t len_elements, size_t elem_bytes, size_t world_size) {
  const int positions = Tunable("IBCOMM_RING_POSITIONS", 4);
  size_t cpr = positions >= 1 && positions <= 64 ? static_cast<size_t>(positions) : 4;
  const int min_env = Tunable("IBCOMM_RING_MIN_CHUNK", 16384);
  const size_t min_chunk = min_env > 0 ? static_cast<size_t>(min_env) : 1;
  const size_t bytes = len_elements * elem_bytes;
  while (cpr > 1 && bytes / (cpr * world_size) < min_chunk) --cpr;
  return cpr;
}

uint64_t TwoShotWindowElems(uint64_t n, uint64_t cap_elems, size_t esize, int world_size, int channels) {
  if (cap_elems == 0) cap_elems = 1;
  if (n <= 1) return 1;
  const uint64_t windows = (n + cap_elems - 1) / cap_elems;
  const uint64_t per = (n + windows - 1) / windows;
  const uint64_t granule = static_cast<uint64_t>(16 / esize) * static_cast<uint64_t>(world_size) * static_cast<uint64_t>(channels > 0 ? channels : 1);
  const uint64_t rounded = (per + granule - 1) / granule * granule;
  // The pool holds a whole number of vectors, so the cap keeps windows aligned.
  return rounded < cap_elems ? rounded : cap_elems;
}

std::string ValidateProgram(const Program& prog, uint64_t len_elements, size_t wire_elem_bytes, int world_size) {
  for (size_t i = 0; i < prog.ops.size(); ++i) {
    const Op& op = prog.ops[i];
    const char* why = nullptr;
    const bool reads_stage = op.src_a == kSrcStage || op.src_b == kSrcStage;
    const bool writes_stage = (op.flags & kOpStoreRemote) != 0;
    if (op.elem_begin > len_elements || op.elem_count > len_elements - op.elem_begin) {
      why = "range outside the message";
    } else if (op.cell_begin > op.elem_begin) {
      why = "cell starts after the range";
    } else if ((reads_stage || writes_stage) &&
               (op.elem_begin - op.cell_begin + op.elem_count) * wire_elem_bytes > prog.stage.slot_bytes) {
      why = "range does not fit its staging slot";
    } else if (reads_stage && (op.region_in >= prog.stage.regions || op.slot_in >= prog.stage.slots)) {
      why = "input slot outside the staging area";
    } else if (writes_stage && (op.region_out >= prog.stage.regions || op.slot_out >= prog.stage.slots)) {
      why = "output slot outside the staging area";
    } else if ((writes_stage || op.wait_credit != 0 || op.post_out != 0) && (op.peer_out < 0 || op.peer_out >= world_size)) {
      why = "peer_out is not a rank";
    } else if ((op.wait_in != 0 || op.post_credit != 0) && (op.peer_in < 0 || op.peer_in >= world_size)) {
      why = "peer_in is not a rank";
    }
    if (why != nullptr) return "op " + std::to_string(i) + ": " + why + ": " + DescribeOp(op);
  }
  return std::string();
}

std::string DescribeOp(const Op& op) {
  static const char* const src[] = {"-", "send", "recv", "stage"};
  char buf[256];
  snprintf(buf, sizeof(buf),
           "[%llu+%llu] a=%s b=%s%s%s%s in=%d(r%u s%u w%u c%u) out=%d(r%u s%u w%u p%u)",
           static_cast<unsigned long long>(op.elem_begin), static_cast<unsigned long long>(op.elem_count),
           src[op.src_a & 3], src[op.src_b & 3], (op.flags & kOpScale) ? " scale" : "",
           (op.flags & kOpStoreLocal) ? " local" : "", (op.flags & kOpStoreRemote) ? " remote" : "", op.peer_in,
           op.region_in, op.slot_in, op.wait_in, op.post_credit, op.peer_out, op.region_out, op.slot_out,
           op.wait_credit, op.post_out);
  return buf;
}

}  // namespace ibcomm
