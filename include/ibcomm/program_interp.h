// Host interpreter of op programs: runs every rank's program on a CPU thread
// against in-memory "arenas" with atomic flags, following the device
// executor's protocol step by step (entry barrier, bounded waits, staging
// slots, credits).  It is the schedule simulator used to validate programs,
// slot/credit accounting and deadlock freedom without a GPU, and it can be
// built with -fsanitize=thread to check the flag protocol for data races.
#pragma once

#include <atomic>
#include <chrono>
#include <cstring>
#include <memory>
#include <thread>
#include <vector>

#include "ibcomm/schedule.h"

namespace ibcomm {

struct SimResult {
  bool ok = true;
  std::string error;
};

template <typename T>
class ProgramSimulator {
 public:
  ProgramSimulator(Algo algo, int world_size, size_t stage_bytes, int channels, size_t piece_elems = 0)
      : algo_(algo), ws_(world_size), stage_bytes_(stage_bytes), nch_(channels), piece_elems_(piece_elems) {}

  // inputs[r] is rank r's send buffer; outputs[r] receives its result.
  // `in_place` makes every rank use one buffer for both.
  SimResult Run(const std::vector<Range>& ranges, const std::vector<std::vector<T>>& inputs,
                std::vector<std::vector<T>>* outputs, double scale, bool in_place, int timeout_ms = 5000) {
    const size_t n = inputs[0].size();
    std::vector<Program> progs;
    for (int r = 0; r < ws_; ++r) {
      ProgramRequest q;
      q.algo = algo_;
      q.rank = r;
      q.world_size = ws_;
      q.ranges = ranges;
      q.piece_elems = piece_elems_;
      q.wire_elem_bytes = sizeof(T);
      q.stage_bytes = stage_bytes_;
      q.apply_scale = (scale != 1.0);
      progs.push_back(BuildProgram(q));
    }
    programs_ = progs;
    const StageLayout st = progs[0].stage;
    struct RankMem {
      std::vector<unsigned char> stage;
      std::unique_ptr<std::atomic<uint64_t>[]> inflag, credit;
    };
    std::vector<RankMem> mem(static_cast<size_t>(ws_));
    for (auto& m : mem) {
      m.stage.assign(static_cast<size_t>(st.regions) * st.slots * st.slot_bytes, 0xAB);
      m.inflag.reset(new std::atomic<uint64_t>[static_cast<size_t>(nch_) * kMaxRanks]);
      m.credit.reset(new std::atomic<uint64_t>[static_cast<size_t>(nch_) * kMaxRanks]);
      for (int i = 0; i < nch_ * kMaxRanks; ++i) {
        m.inflag[static_cast<size_t>(i)].store(0);
        m.credit[static_cast<size_t>(i)].store(0);
      }
    }
    outputs->assign(static_cast<size_t>(ws_), std::vector<T>());
    for (int r = 0; r < ws_; ++r) (*outputs)[static_cast<size_t>(r)] = in_place ? inputs[static_cast<size_t>(r)] : std::vector<T>(n, T(-77));

    std::atomic<bool> abort{false};
    std::vector<std::string> errors(static_cast<size_t>(ws_) * static_cast<size_t>(nch_));
    auto worker = [&](int r, int ch) {
      const Program& pg = progs[static_cast<size_t>(r)];
      const T* sendbuf = in_place ? (*outputs)[static_cast<size_t>(r)].data() : inputs[static_cast<size_t>(r)].data();
      T* recvbuf = (*outputs)[static_cast<size_t>(r)].data();
      auto wait_for = [&](std::atomic<uint64_t>& f, uint64_t target, const char* what, size_t op_index) {
        auto t0 = std::chrono::steady_clock::now();
        unsigned spins = 0;
        while (f.load(std::memory_order_acquire) < target) {
          if (abort.load()) return false;
          if ((++spins & 0xff) == 0) {
            std::this_thread::yield();
            if (std::chrono::steady_clock::now() - t0 > std::chrono::milliseconds(timeout_ms)) {
              errors[static_cast<size_t>(r * nch_ + ch)] = std::string("rank ") + std::to_string(r) + " ch " + std::to_string(ch) +
                                                           " op " + std::to_string(op_index) + " timed out waiting for " + what +
                                                           " >= " + std::to_string(target) + " (" + DescribeOp(pg.ops[op_index]) + ")";
              abort.store(true);
              return false;
            }
          }
        }
        return true;
      };
      for (size_t oi = 0; oi < pg.ops.size(); ++oi) {
        const Op& op = pg.ops[oi];
        uint64_t lo, hi;
        ChannelSlice(op.elem_begin - op.cell_begin, op.elem_count, st.slot_bytes / sizeof(T), nch_, ch, &lo, &hi);
        RankMem& me = mem[static_cast<size_t>(r)];
        if (op.wait_in != 0 &&
            !wait_for(me.inflag[static_cast<size_t>(ch * kMaxRanks + op.peer_in)], op.wait_in, "data", oi))
          return;
        if (op.wait_credit != 0 &&
            !wait_for(me.credit[static_cast<size_t>(ch * kMaxRanks + op.peer_out)], op.wait_credit, "credit", oi))
          return;
        const T* stage_in = nullptr;
        if (op.src_a == kSrcStage)
          stage_in = reinterpret_cast<const T*>(me.stage.data() + (static_cast<size_t>(op.region_in) * st.slots + op.slot_in) * st.slot_bytes);
        T* stage_out = nullptr;
        if (op.flags & kOpStoreRemote)
          stage_out = reinterpret_cast<T*>(mem[static_cast<size_t>(op.peer_out)].stage.data() +
                                           (static_cast<size_t>(op.region_out) * st.slots + op.slot_out) * st.slot_bytes);
        for (uint64_t k = lo; k < hi; ++k) {
          const uint64_t g = op.cell_begin + k;
          T v = op.src_a == kSrcStage ? stage_in[k] : (op.src_a == kSrcSend ? sendbuf[g] : recvbuf[g]);
          if (op.src_b == kSrcSend) v = static_cast<T>(v + sendbuf[g]);
          else if (op.src_b == kSrcRecv) v = static_cast<T>(v + recvbuf[g]);
          if (op.flags & kOpScale) v = static_cast<T>(v * scale);
          if (op.flags & kOpStoreLocal) recvbuf[g] = v;
          if (stage_out != nullptr) stage_out[k] = v;
        }
        if (op.post_out != 0)
          mem[static_cast<size_t>(op.peer_out)].inflag[static_cast<size_t>(ch * kMaxRanks + r)].store(op.post_out, std::memory_order_release);
        if (op.post_credit != 0)
          mem[static_cast<size_t>(op.peer_in)].credit[static_cast<size_t>(ch * kMaxRanks + r)].store(op.post_credit, std::memory_order_release);
      }
    };
    std::vector<std::thread> threads;
    for (int r = 0; r < ws_; ++r)
      for (int ch = 0; ch < nch_; ++ch) threads.emplace_back(worker, r, ch);
    for (auto& t : threads) t.join();
    SimResult res;
    for (const std::string& e : errors)
      if (!e.empty()) {
        res.ok = false;
        res.error += e + "\n";
      }
    return res;
  }

  const std::vector<Program>& programs() const { return programs_; }

 private:
  Algo algo_;
  int ws_;
  size_t stage_bytes_;
  int nch_;
  size_t piece_elems_;
  std::vector<Program> programs_;
};

}  // namespace ibcomm
