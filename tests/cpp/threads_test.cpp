// Single-process model: N host threads, one communicator each (and, with
// `cuda`, one GPU each), connected through the three-call protocol with the
// descriptors handed over in process memory.  The reference only ever runs one
// rank per process (examples/allreduce.cpp:38-77); this is the second process
// model the library supports.
//
//   threads_test cpu  <ranks>      host buffers over the shared-memory rings
//   threads_test cuda <ranks>      device buffers, rank r on GPU r
//
// Prints "threads_test OK" and exits 0 when every rank's result matches.
#include <atomic>
#include <cmath>
#include <condition_variable>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include "ibcomm/communicator.h"
#ifdef USE_CUDA
#include <cuda_runtime.h>

#include "ibcomm/memory_pool.h"
#endif

namespace {

class ThreadBarrier {
 public:
  explicit ThreadBarrier(int n) : n_(n) {}
  void Wait() {
    std::unique_lock<std::mutex> lk(mu_);
    const int gen = gen_;
    if (++count_ == n_) {
      count_ = 0;
      ++gen_;
      cv_.notify_all();
    } else {
      cv_.wait(lk, [&] { return gen != gen_; });
    }
  }

 private:
  std::mutex mu_;
  std::condition_variable cv_;
  int n_, count_ = 0, gen_ = 0;
};

float Value(int rank, size_t i) { return static_cast<float>((static_cast<long long>(i % 1013) - 500) * (rank + 1)) * 0.25f; }

float Expected(int ws, size_t i) {
  float s = 0;
  for (int r = 0; r < ws; ++r) s += Value(r, i);
  return s;
}

size_t CountBad(const std::vector<float>& out, int ws, double scale) {
  size_t bad = 0;
  for (size_t i = 0; i < out.size(); ++i)
    if (std::fabs(out[i] - Expected(ws, i) * scale) > 1e-3) ++bad;
  return bad;
}

}  // namespace

#ifdef USE_CUDA
// The staging pool with pinned blocks and CUDA streams: six slots in flight,
// each copied to the device on the stream it was handed out with; six at once
// need a second block (four slots each) and two streams beyond the first four.
int PoolOnDevice() {
  constexpr size_t kSlot = 256u << 10;
  ibcomm::MemoryPool<ibcomm::PinnedBlockAllocator, ibcomm::CudaStreams> pool(1 << 20, 4);
  auto ctl = pool.GetController(kSlot);
  unsigned char* dev = nullptr;
  if (cudaMalloc(&dev, 6 * kSlot) != cudaSuccess) return 3;
  std::vector<ibcomm::Memory*> out;
  for (int i = 0; i < 6; ++i) {
    ibcomm::Memory* m = ctl.getMemory();
    memset(m->ptr(), 0x10 + i, kSlot);
    cudaMemcpyAsync(dev + i * kSlot, m->ptr(), kSlot, cudaMemcpyHostToDevice, static_cast<cudaStream_t>(m->stream()));
    out.push_back(m);
  }
  int bad = 0;
  for (int i = 0; i < 6; ++i) {
    if (cudaStreamSynchronize(static_cast<cudaStream_t>(out[i]->stream())) != cudaSuccess) ++bad;
    ctl.returnMemory(out[i]);
  }
  std::vector<unsigned char> back(6 * kSlot);
  if (cudaMemcpy(back.data(), dev, back.size(), cudaMemcpyDeviceToHost) != cudaSuccess) ++bad;
  for (int i = 0; i < 6; ++i)
    if (back[i * kSlot] != 0x10 + i || back[(i + 1) * kSlot - 1] != 0x10 + i) ++bad;
  cudaFree(dev);
  if (pool.num_blocks() != 2 || pool.num_streams() != 6 || ctl.vacant_slots() != 8) ++bad;
  printf(bad == 0 ? "pool OK\n" : "pool FAILED\n");
  return bad == 0 ? 0 : 1;
}
#endif

int main(int argc, char** argv) {
  const std::string device = argc > 1 ? argv[1] : "cpu";
#ifdef USE_CUDA
  if (device == "pool") return PoolOnDevice();
#endif
  const int ws = argc > 2 ? atoi(argv[2]) : 2;
  if (ws < 1 || ws > 8 || (device != "cpu" && device != "cuda")) {
    fprintf(stderr, "usage: threads_test cpu|cuda <ranks 1..8>\n");
    return 1;
  }
#ifndef USE_CUDA
  if (device == "cuda") {
    fprintf(stderr, "threads_test: built without CUDA\n");
    return 4;
  }
#else
  if (device == "cuda") {
    int ngpu = 0;
    if (cudaGetDeviceCount(&ngpu) != cudaSuccess || ngpu < ws) {
      fprintf(stderr, "threads_test: %d GPUs needed, %d found\n", ws, ngpu);
      return 4;
    }
  }
#endif
  std::vector<std::vector<ProcessInfo>> infos(static_cast<size_t>(ws), std::vector<ProcessInfo>(static_cast<size_t>(ws)));
  ThreadBarrier barrier(ws);
  std::atomic<size_t> bad{0};

  auto body = [&](int rank) {
#ifdef USE_CUDA
    if (device == "cuda") cudaSetDevice(rank);
#endif
    ibcomm::Communicator comm(ws);
    for (int q = 0; q < ws; ++q)
      if (q != rank) infos[static_cast<size_t>(rank)][static_cast<size_t>(q)] = comm.CreateQueuePair(q);
    barrier.Wait();
    for (int q = 0; q < ws; ++q)
      if (q != rank) comm.RegisterQueuePair(q, infos[static_cast<size_t>(q)][static_cast<size_t>(rank)]);
    comm.RegisterMyself(rank);
    barrier.Wait();

    for (size_t n : {static_cast<size_t>(ws), static_cast<size_t>(1000), (static_cast<size_t>(1) << 20) + 3}) {
      std::vector<float> in(n), out(n, -1.0f);
      for (size_t i = 0; i < n; ++i) in[i] = Value(rank, i);
      if (device == "cpu") {
        comm.AllreduceRing(in.data(), out.data(), n);
        bad += CountBad(out, ws, 1.0);
        if (ws > 1) {
          std::fill(out.begin(), out.end(), -1.0f);
          comm.AllreduceRabenseifner(in.data(), out.data(), n);
          bad += CountBad(out, ws, 1.0);
        }
      } else {
#ifdef USE_CUDA
        float *d_in = nullptr, *d_out = nullptr;
        cudaMalloc(&d_in, n * sizeof(float));
        cudaMalloc(&d_out, n * sizeof(float));
        cudaMemcpy(d_in, in.data(), n * sizeof(float), cudaMemcpyHostToDevice);
        comm.AllreduceRingCuda(d_in, d_out, n);
        cudaMemcpy(out.data(), d_out, n * sizeof(float), cudaMemcpyDeviceToHost);
        bad += CountBad(out, ws, 1.0);
        comm.AllreduceRabenseifnerCuda(d_in, d_out, n);
        cudaMemcpy(out.data(), d_out, n * sizeof(float), cudaMemcpyDeviceToHost);
        bad += CountBad(out, ws, 1.0);
        ibcomm::CudaAllreduceOptions o;  // algorithm by size, fused scale
        o.scale = 0.5;
        cudaMemset(d_out, 0, n * sizeof(float));
        comm.AllreduceCuda(ibcomm::DType::kFloat32, d_in, d_out, n, o);
        cudaMemcpy(out.data(), d_out, n * sizeof(float), cudaMemcpyDeviceToHost);
        bad += CountBad(out, ws, 0.5);
        cudaFree(d_in);
        cudaFree(d_out);
#endif
      }
    }
    // Nobody tears its endpoints down while a peer may still read them.
    barrier.Wait();
  };

  std::vector<std::thread> threads;
  for (int r = 0; r < ws; ++r) threads.emplace_back(body, r);
  for (std::thread& t : threads) t.join();
  if (bad.load() != 0) {
    fprintf(stderr, "threads_test: %zu wrong elements\n", bad.load());
    return 1;
  }
  printf("threads_test OK (%s, %d ranks)\n", device.c_str(), ws);
  return 0;
}
