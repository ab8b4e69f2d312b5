#include "ibcomm/c_api.h"

#include <cstring>
#include <string>
#include <vector>

#include "ibcomm/communicator.h"
#include "ibcomm/device_context.h"
#include "ibcomm/schedule.h"
#include "ibcomm/tunables.h"
#ifdef USE_CUDA
#include <cuda_runtime.h>

#include "ibcomm/emu_world.h"
#include "kernels.h"
#endif

using ibcomm::Communicator;

struct ibcomm_comm {
  Communicator comm;
};
#ifdef USE_CUDA
struct ibcomm_emu {
  explicit ibcomm_emu(int n, size_t pool, size_t work) : world(n, pool, work) {}
  ibcomm::EmuWorld world;
};
#else
struct ibcomm_emu {
  int unused;
};
#endif

namespace {

thread_local std::string g_last_error;

template <typename Fn>
int Guard(Fn fn) {
  ibcomm::SetErrorPolicy(ibcomm::ErrorPolicy::kThrow);
  try {
    fn();
    return 0;
  } catch (const ibcomm::Error& e) {
    g_last_error = e.what();
    return e.code();
  } catch (const std::exception& e) {
    g_last_error = e.what();
    return 1;
  }
}

ProcessInfo FromWords(const uint32_t w[3]) {
  ProcessInfo p;
  p.lid = static_cast<uint16_t>(w[0]);
  p.qp_n = w[1];
  p.psn = w[2];
  return p;
}
void ToWords(const ProcessInfo& p, uint32_t w[3]) {
  w[0] = p.lid;
  w[1] = p.qp_n;
  w[2] = p.psn;
}

ibcomm::DType CheckDType(int d) {
  if (d < 0 || d > 5) IBCOMM_FAIL(INVALID_ARGUMENT, "Unknown dtype code %d.\n", d);
  return static_cast<ibcomm::DType>(d);
}
ibcomm::Algo CheckAlgo(int a) {
  if (a < 0 || a > 5) IBCOMM_FAIL(INVALID_ARGUMENT, "Unknown algorithm code %d.\n", a);
  return static_cast<ibcomm::Algo>(a);
}

// A destroyed (or never created) handle is an argument error, not a crash.
void NeedHandle(const void* h) {
  if (h == nullptr) IBCOMM_FAIL(INVALID_ARGUMENT, "The handle is null (already destroyed?).\n");
}

[[maybe_unused]] void NeedCuda() {
#ifndef USE_CUDA
  IBCOMM_FAIL(NOT_SUPPORTED, "This build of the library has no CUDA support.\n");
#endif
}

}  // namespace

extern "C" {

const char* ibcomm_last_error(void) { return g_last_error.c_str(); }

int ibcomm_has_cuda(void) {
#ifdef USE_CUDA
  return 1;
#else
  return 0;
#endif
}

int ibcomm_create(int world_size, ibcomm_comm** out) {
  return Guard([&] {
    if (out == nullptr) IBCOMM_FAIL(INVALID_ARGUMENT, "out is null.\n");
    ibcomm_comm* c = new ibcomm_comm();
    try {
      c->comm.Init(world_size);
    } catch (...) {
      delete c;
      throw;
    }
    *out = c;
  });
}

int ibcomm_destroy(ibcomm_comm* c) {
  return Guard([&] {
    NeedHandle(c);
    delete c;
  });
}

int ibcomm_create_queue_pair(ibcomm_comm* c, int dest_rank, uint32_t info_out[3]) {
  return Guard([&] {
    NeedHandle(c);
    ToWords(c->comm.CreateQueuePair(dest_rank), info_out);
  });
}
int ibcomm_register_queue_pair(ibcomm_comm* c, int dest_rank, const uint32_t info[3]) {
  return Guard([&] {
    NeedHandle(c);
    c->comm.RegisterQueuePair(dest_rank, FromWords(info));
  });
}
int ibcomm_register_process(ibcomm_comm* c, int dest_rank, const uint32_t info[3], uint32_t info_out[3]) {
  return Guard([&] {
    NeedHandle(c);
    ToWords(c->comm.RegisterProcess(dest_rank, FromWords(info)), info_out);
  });
}
int ibcomm_register_myself(ibcomm_comm* c, int my_rank) {
  return Guard([&] {
    NeedHandle(c);
    c->comm.RegisterMyself(my_rank);
  });
}
int ibcomm_set_timeout_ms(ibcomm_comm* c, int ms) {
  return Guard([&] {
    NeedHandle(c);
    c->comm.SetTimeoutMs(ms);
  });
}

int ibcomm_set_max_channels(ibcomm_comm* c, int channels) {
  return Guard([&] {
    NeedHandle(c);
    NeedCuda();
#ifdef USE_CUDA
    c->comm.PrepareMemoryPool();
    ibcomm::DeviceContextSetMaxChannels(c->comm.device(), channels);
#else
    (void)c; (void)channels;
#endif
  });
}

int ibcomm_send(ibcomm_comm* c, int dest_rank, const void* buf, size_t len, int blocking) {
  return Guard([&] {
    NeedHandle(c);
    c->comm.Send(dest_rank, buf, len, blocking != 0);
  });
}
int ibcomm_recv(ibcomm_comm* c, int src_rank, void* buf, size_t len, int blocking) {
  return Guard([&] {
    NeedHandle(c);
    c->comm.Recv(src_rank, buf, len, blocking != 0);
  });
}
int ibcomm_send_poll(ibcomm_comm* c, int dest_rank, int* done) {
  return Guard([&] {
    NeedHandle(c);
    *done = c->comm.SendPoll(dest_rank) ? 1 : 0;
  });
}
int ibcomm_recv_poll(ibcomm_comm* c, int src_rank, int* done) {
  return Guard([&] {
    NeedHandle(c);
    *done = c->comm.RecvPoll(src_rank) ? 1 : 0;
  });
}
int ibcomm_send_wait(ibcomm_comm* c, int dest_rank) {
  return Guard([&] {
    NeedHandle(c);
    c->comm.SendWait(dest_rank);
  });
}
int ibcomm_recv_wait(ibcomm_comm* c, int src_rank) {
  return Guard([&] {
    NeedHandle(c);
    c->comm.RecvWait(src_rank);
  });
}
int ibcomm_bcast(ibcomm_comm* c, void* buf, size_t len, int root) {
  return Guard([&] {
    NeedHandle(c);
    c->comm.Bcast(buf, len, root);
  });
}
int ibcomm_barrier(ibcomm_comm* c) {
  return Guard([&] {
    NeedHandle(c);
    c->comm.Barrier();
  });
}

int ibcomm_allreduce_host(ibcomm_comm* c, int algo, int dtype, const void* sendbuf, void* recvbuf, size_t n) {
  return Guard([&] {
    NeedHandle(c);
    const ibcomm::Algo a = CheckAlgo(algo);
    const ibcomm::DType d = CheckDType(dtype);
    if (a != ibcomm::Algo::kRing && a != ibcomm::Algo::kRabenseifner)
      IBCOMM_FAIL(INVALID_ARGUMENT, "Host buffers support the ring and rabenseifner algorithms.\n");
    const bool ring = a == ibcomm::Algo::kRing;
    Communicator& m = c->comm;
#define IBCOMM_HOST_CASE(T)                                                                   \
  do {                                                                                        \
    if (ring) m.AllreduceRing(static_cast<const T*>(sendbuf), static_cast<T*>(recvbuf), n);   \
    else m.AllreduceRabenseifner(static_cast<const T*>(sendbuf), static_cast<T*>(recvbuf), n); \
  } while (0)
    switch (d) {
      case ibcomm::DType::kFloat32: IBCOMM_HOST_CASE(float); break;
      case ibcomm::DType::kFloat64: IBCOMM_HOST_CASE(double); break;
      case ibcomm::DType::kInt32: IBCOMM_HOST_CASE(int32_t); break;
      case ibcomm::DType::kInt64: IBCOMM_HOST_CASE(int64_t); break;
      default: IBCOMM_FAIL(NOT_SUPPORTED, "Host allreduce supports float32, float64, int32 and int64.\n");
    }
#undef IBCOMM_HOST_CASE
  });
}

static int HostRsAg(ibcomm_comm* c, bool all_gather, int dtype, const void* sendbuf, void* recvbuf, size_t block_elements) {
  return Guard([&] {
    Communicator& m = c->comm;
#define IBCOMM_HOST_CASE(T)                                                                               \
  do {                                                                                                    \
    if (all_gather) m.AllGather(static_cast<const T*>(sendbuf), static_cast<T*>(recvbuf), block_elements); \
    else m.ReduceScatter(static_cast<const T*>(sendbuf), static_cast<T*>(recvbuf), block_elements);       \
  } while (0)
    switch (CheckDType(dtype)) {
      case ibcomm::DType::kFloat32: IBCOMM_HOST_CASE(float); break;
      case ibcomm::DType::kFloat64: IBCOMM_HOST_CASE(double); break;
      case ibcomm::DType::kInt32: IBCOMM_HOST_CASE(int32_t); break;
      case ibcomm::DType::kInt64: IBCOMM_HOST_CASE(int64_t); break;
      default: IBCOMM_FAIL(NOT_SUPPORTED, "Host reduce-scatter / all-gather support float32, float64, int32 and int64.\n");
    }
#undef IBCOMM_HOST_CASE
  });
}

int ibcomm_reduce_scatter_host(ibcomm_comm* c, int dtype, const void* sendbuf, void* recvbuf, size_t block_elements) {
  return HostRsAg(c, false, dtype, sendbuf, recvbuf, block_elements);
}

int ibcomm_all_gather_host(ibcomm_comm* c, int dtype, const void* sendbuf, void* recvbuf, size_t block_elements) {
  return HostRsAg(c, true, dtype, sendbuf, recvbuf, block_elements);
}

int ibcomm_allreduce_cuda(ibcomm_comm* c, int algo, int dtype, const void* sendbuf, void* recvbuf, size_t n, double scale,
                          int wire_dtype, void* stream, int flags) {
  return Guard([&] {
    NeedHandle(c);
    NeedCuda();
#ifdef USE_CUDA
    ibcomm::CudaAllreduceOptions o;
    o.algo = CheckAlgo(algo);
    o.scale = scale;
    o.wire = CheckDType(wire_dtype);
    o.stream = stream;
    o.use_stream = (flags & IBCOMM_USE_STREAM) != 0;
    o.async = (flags & IBCOMM_ASYNC) != 0;
    c->comm.AllreduceCuda(CheckDType(dtype), sendbuf, recvbuf, n, o);
#else
    (void)c; (void)algo; (void)dtype; (void)sendbuf; (void)recvbuf; (void)n; (void)scale; (void)wire_dtype; (void)stream; (void)flags;
#endif
  });
}

int ibcomm_reduce_scatter_cuda(ibcomm_comm* c, int algo, int dtype, const void* sendbuf, void* recvbuf, size_t block_elements,
                               double scale, void* stream, int flags) {
  return Guard([&] {
    NeedHandle(c);
    NeedCuda();
#ifdef USE_CUDA
    ibcomm::CudaAllreduceOptions o;
    o.algo = CheckAlgo(algo);
    o.scale = scale;
    o.stream = stream;
    o.use_stream = (flags & IBCOMM_USE_STREAM) != 0;
    o.async = (flags & IBCOMM_ASYNC) != 0;
    c->comm.ReduceScatterCuda(CheckDType(dtype), sendbuf, recvbuf, block_elements, o);
#else
    (void)c; (void)algo; (void)dtype; (void)sendbuf; (void)recvbuf; (void)block_elements; (void)scale; (void)stream; (void)flags;
#endif
  });
}

int ibcomm_all_gather_cuda(ibcomm_comm* c, int algo, int dtype, const void* sendbuf, void* recvbuf, size_t block_elements,
                           void* stream, int flags) {
  return Guard([&] {
    NeedHandle(c);
    NeedCuda();
#ifdef USE_CUDA
    ibcomm::CudaAllreduceOptions o;
    o.algo = CheckAlgo(algo);
    o.stream = stream;
    o.use_stream = (flags & IBCOMM_USE_STREAM) != 0;
    o.async = (flags & IBCOMM_ASYNC) != 0;
    c->comm.AllGatherCuda(CheckDType(dtype), sendbuf, recvbuf, block_elements, o);
#else
    (void)c; (void)algo; (void)dtype; (void)sendbuf; (void)recvbuf; (void)block_elements; (void)stream; (void)flags;
#endif
  });
}

int ibcomm_choose_algorithm(size_t bytes, int world_size, int nvls, int mapped, int max_channels, int* algo, int* channels) {
  return Guard([&] {
    if (world_size < 1 || world_size > ibcomm::kMaxRanks || algo == nullptr || channels == nullptr)
      IBCOMM_FAIL(INVALID_ARGUMENT, "ibcomm_choose_algorithm: world size 1..%d and two result pointers.\n", ibcomm::kMaxRanks);
    const ibcomm::TunerChoice c = ibcomm::ChooseAlgorithm(bytes, world_size, nvls != 0, mapped != 0,
                                                          max_channels > 0 ? max_channels : ibcomm::kMaxChannels);
    *algo = static_cast<int>(c.algo);
    *channels = c.channels;
  });
}

int ibcomm_check(ibcomm_comm* c) {
  return Guard([&] {
    NeedHandle(c);
#ifdef USE_CUDA
    if (c->comm.device() != nullptr) ibcomm::DeviceContextCheck(c->comm.device());
#else
    (void)c;
#endif
  });
}

int ibcomm_symmetric_alloc(ibcomm_comm* c, size_t bytes, void** out) {
  return Guard([&] {
    NeedHandle(c);
    NeedCuda();
#ifdef USE_CUDA
    *out = ibcomm::DeviceContextSymmetricAlloc(&c->comm, bytes);
#else
    (void)c; (void)bytes; (void)out;
#endif
  });
}

int ibcomm_symmetric_free(ibcomm_comm* c, void* ptr) {
  return Guard([&] {
    NeedHandle(c);
    NeedCuda();
#ifdef USE_CUDA
    ibcomm::DeviceContextSymmetricFree(&c->comm, ptr);
#else
    (void)c; (void)ptr;
#endif
  });
}

int ibcomm_register_buffer(ibcomm_comm* c, void* ptr, size_t bytes, int* id) {
  return Guard([&] {
    NeedHandle(c);
    NeedCuda();
#ifdef USE_CUDA
    *id = ibcomm::DeviceContextRegisterBuffer(&c->comm, ptr, bytes);
#else
    (void)c; (void)ptr; (void)bytes; (void)id;
#endif
  });
}

int ibcomm_deregister_buffer(ibcomm_comm* c, int id) {
  return Guard([&] {
    NeedHandle(c);
    NeedCuda();
#ifdef USE_CUDA
    ibcomm::DeviceContextDeregisterBuffer(&c->comm, id);
#else
    (void)c; (void)id;
#endif
  });
}

int ibcomm_get_device_info(ibcomm_comm* c, int connect, ibcomm_device_info* out) {
  return Guard([&] {
    NeedHandle(c);
    NeedCuda();
#ifdef USE_CUDA
    c->comm.PrepareMemoryPool();
    if (connect) {
      // The first collective connects the peers; a tiny symmetric allocation
      // does the same without moving data.
      void* p = ibcomm::DeviceContextSymmetricAlloc(&c->comm, 4096);
      ibcomm::DeviceContextSymmetricFree(&c->comm, p);
    }
    ibcomm::DeviceInfo i = ibcomm::DeviceContextInfo(c->comm.device());
    memset(out, 0, sizeof(*out));
    out->device = i.device;
    out->nvls = i.nvls;
    out->share_mode = i.share_mode;
    out->last_algo = i.last_algo;
    out->last_channels = i.last_channels;
    out->arena_bytes = i.arena_bytes;
    out->pool_bytes = i.pool_bytes;
    out->work_bytes = i.work_bytes;
    out->calls = i.calls;
    out->kernel_launches = i.kernel_launches;
    out->switch_registrations = i.switch_registrations;
#else
    (void)c; (void)connect; (void)out;
#endif
  });
}

int ibcomm_set_timer_base(ibcomm_comm* c) {
  return Guard([&] {
    NeedHandle(c);
    c->comm.SetTimerBase();
  });
}
int ibcomm_dump_trace(ibcomm_comm* c) {
  return Guard([&] {
    NeedHandle(c);
    c->comm.DumpTrace();
  });
}
int ibcomm_staged_timeline(ibcomm_comm* c, uint64_t* out, size_t capacity_words, size_t* words) {
  return Guard([&] {
    NeedHandle(c);
    *words = 0;
#ifdef USE_CUDA
    if (c->comm.device() != nullptr) {
      ibcomm::DeviceContextCollectTrace(c->comm.device(), &c->comm.tracer());
      *words = ibcomm::DeviceContextStagedTimeline(c->comm.device(), out, capacity_words);
    }
#else
    (void)out; (void)capacity_words;
#endif
  });
}

int ibcomm_emu_create(int num_ranks, size_t pool_bytes, size_t work_bytes, ibcomm_emu** out) {
  return Guard([&] {
    NeedCuda();
#ifdef USE_CUDA
    *out = new ibcomm_emu(num_ranks, pool_bytes, work_bytes);
#else
    (void)num_ranks; (void)pool_bytes; (void)work_bytes; (void)out;
#endif
  });
}

int ibcomm_emu_destroy(ibcomm_emu* w) {
  return Guard([&] {
    NeedHandle(w);
    delete w;
  });
}

int ibcomm_emu_allreduce(ibcomm_emu* w, int algo, int dtype, const void* const* sendbufs, void* const* recvbufs, size_t n,
                         double scale, int wire_dtype, int channels, void* stream, int async) {
  return Guard([&] {
    NeedHandle(w);
    NeedCuda();
#ifdef USE_CUDA
    const int ws = w->world.num_ranks();
    std::vector<const void*> in(sendbufs, sendbufs + ws);
    std::vector<void*> out(recvbufs, recvbufs + ws);
    w->world.Allreduce(CheckAlgo(algo), CheckDType(dtype), in, out, n, scale, CheckDType(wire_dtype), channels, stream, async != 0);
#else
    (void)w; (void)algo; (void)dtype; (void)sendbufs; (void)recvbufs; (void)n; (void)scale; (void)wire_dtype; (void)channels; (void)stream; (void)async;
#endif
  });
}

int ibcomm_emu_rsag(ibcomm_emu* w, int all_gather, int dtype, const void* const* sendbufs, void* const* recvbufs,
                    size_t block_elements, double scale, int channels, void* stream, int async) {
  return Guard([&] {
    NeedHandle(w);
    NeedCuda();
#ifdef USE_CUDA
    const int ws = w->world.num_ranks();
    std::vector<const void*> in(sendbufs, sendbufs + ws);
    std::vector<void*> out(recvbufs, recvbufs + ws);
    w->world.ReduceScatterOrAllGather(all_gather != 0, CheckDType(dtype), in, out, block_elements, scale, channels, stream, async != 0);
#else
    (void)w; (void)all_gather; (void)dtype; (void)sendbufs; (void)recvbufs; (void)block_elements; (void)scale; (void)channels; (void)stream; (void)async;
#endif
  });
}

int ibcomm_emu_set_timeout_ms(ibcomm_emu* w, int ms) {
  return Guard([&] {
    NeedHandle(w);
#ifdef USE_CUDA
    w->world.SetTimeoutMs(ms);
#else
    (void)w; (void)ms;
#endif
  });
}

int ibcomm_emu_last_channels(ibcomm_emu* w) {
#ifdef USE_CUDA
  return w->world.last_channels();
#else
  (void)w;
  return 0;
#endif
}

int ibcomm_emu_set_bad_program_rank(ibcomm_emu* w, int rank) {
  return Guard([&] {
    NeedHandle(w);
#ifdef USE_CUDA
    w->world.SetBadProgramRank(rank);
#else
    (void)w; (void)rank;
#endif
  });
}

int ibcomm_emu_set_silent_rank(ibcomm_emu* w, int rank) {
  return Guard([&] {
    NeedHandle(w);
#ifdef USE_CUDA
    w->world.SetSilentRank(rank);
#else
    (void)w; (void)rank;
#endif
  });
}

int ibcomm_emu_set_direct_staging(ibcomm_emu* w, int on) {
  return Guard([&] {
    NeedHandle(w);
#ifdef USE_CUDA
    w->world.SetDirectStaging(on);
#else
    (void)w; (void)on;
#endif
  });
}

int ibcomm_emu_last_status(ibcomm_emu* w, ibcomm_status_report* out) {
  return Guard([&] {
    NeedHandle(w);
#ifdef USE_CUDA
    ibcomm::DeviceStatus st;
    memset(&st, 0, sizeof(st));
    uint32_t code = w->world.LastStatus(&st);
    static_assert(sizeof(ibcomm_status_report) == sizeof(ibcomm::DeviceStatus), "status layouts must match");
    memcpy(out, &st, sizeof(st));
    out->code = code;
#else
    (void)w; (void)out;
#endif
  });
}

int ibcomm_copy_scale(const void* in, void* out, size_t n, int dtype_in, int dtype_out, double scale, void* stream) {
  return Guard([&] {
    NeedCuda();
#ifdef USE_CUDA
    ibcomm::CopyParams p{in, out, n, static_cast<int32_t>(CheckDType(dtype_in)), static_cast<int32_t>(CheckDType(dtype_out)), scale};
    cudaError_t e = ibcomm::LaunchCopyKernel(p, ibcomm::kCopyDefaultBlocks, static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) IBCOMM_FAIL(CUDA_ERROR, "copy kernel launch failed: %s\n", cudaGetErrorString(e));
#else
    (void)in; (void)out; (void)n; (void)dtype_in; (void)dtype_out; (void)scale; (void)stream;
#endif
  });
}

int ibcomm_parse_number(const char* text, int64_t* out) {
  try {
    *out = util::parse_number(text ? text : "");
    return 0;
  } catch (const util::MalformedNumber& e) {
    g_last_error = e.what();
    return 1;
  }
}

int ibcomm_get_exp_of_two(uint64_t n) { return util::GetExpOfTwo(n); }

int ibcomm_set_tunable(const char* name, int value) {
  return Guard([&] {
    if (name == nullptr || name[0] == '\0') IBCOMM_FAIL(INVALID_ARGUMENT, "ibcomm_set_tunable: empty name.\n");
    ibcomm::SetTunable(name, value);
  });
}

int ibcomm_get_tunable(const char* name, int dflt, int* out) {
  return Guard([&] {
    if (name == nullptr || out == nullptr) IBCOMM_FAIL(INVALID_ARGUMENT, "ibcomm_get_tunable: null argument.\n");
    *out = ibcomm::Tunable(name, dflt);
  });
}

int ibcomm_split_buffer(size_t len_elements, size_t elem_bytes, size_t world_size, int64_t chunk_bytes, uint64_t* pairs,
                        size_t capacity, size_t* count) {
  return Guard([&] {
    std::vector<ibcomm::Range> r = ibcomm::SplitBuffer(len_elements, elem_bytes, world_size, chunk_bytes);
    *count = r.size();
    for (size_t i = 0; i < r.size() && i < capacity; ++i) {
      pairs[2 * i] = r[i].first;
      pairs[2 * i + 1] = r[i].second;
    }
  });
}

int ibcomm_rank_to_chunk(size_t num_chunks, size_t world_size, int rank, int* chunks, size_t capacity, size_t* count) {
  return Guard([&] {
    auto m = ibcomm::GetRankToChunk(num_chunks, world_size);
    if (rank < 0 || static_cast<size_t>(rank) >= m.size()) IBCOMM_FAIL(INVALID_ARGUMENT, "rank out of range.\n");
    const auto& v = m[static_cast<size_t>(rank)];
    *count = v.size();
    for (size_t i = 0; i < v.size() && i < capacity; ++i) chunks[i] = v[i];
  });
}

int ibcomm_describe_program(int algo, int rank, int world_size, size_t len_elements, size_t elem_bytes, int64_t chunk_bytes,
                            size_t stage_bytes, char* text, size_t capacity) {
  return Guard([&] {
    ibcomm::ProgramRequest q;
    q.algo = CheckAlgo(algo);
    q.rank = rank;
    q.world_size = world_size;
    q.ranges = ibcomm::SplitForDevice(len_elements, elem_bytes, static_cast<size_t>(world_size), chunk_bytes, 0);
    q.wire_elem_bytes = elem_bytes;
    q.stage_bytes = stage_bytes;
    ibcomm::Program p = ibcomm::BuildProgram(q);
    std::string s;
    for (const ibcomm::Op& op : p.ops) s += ibcomm::DescribeOp(op) + "\n";
    if (capacity > 0) {
      size_t n = s.size() < capacity - 1 ? s.size() : capacity - 1;
      memcpy(text, s.data(), n);
      text[n] = '\0';
    }
  });
}

}  // extern "C"
