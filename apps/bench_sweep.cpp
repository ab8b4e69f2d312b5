// bench_sweep — message-size sweep of the device allreduce from C++ (no Python,
// no NCCL): one JSON line per size and algorithm on rank 0.
//
//   ibcomm_run -np 8 build/bin/bench_sweep [--min 4k] [--max 1g] [--algos auto,ring,...]
//              [--symmetric 0|1] [--op allreduce|reduce_scatter|all_gather]
//
// The reference's only benchmark is its example (examples/allreduce.cpp:96-146:
// one size, host wall clock of the last of four runs on rank 0).  Here every
// size from --min to --max (powers of two) is timed on the device: CUDA events
// on the stream of the calls around `iters` asynchronous calls after `warm`
// warm-up calls, a host barrier and a device synchronise on both sides, the
// maximum over the ranks.  Bus bandwidth = bytes / time x 2 (N-1) / N for the
// allreduce, x (N-1) / N for its halves (bytes = the full buffer).
// --symmetric 1 (default) takes the buffers from the communicator's peer-mapped
// memory (zero-copy paths); 0 uses plain cudaMalloc memory, registered with the
// communicator when --register 1 is given.
#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <sstream>
#include <string>
#include <vector>

#include "ibcomm/bootstrap.h"
#include "ibcomm/communicator.h"
#include "ibcomm/device_context.h"

#ifndef USE_CUDA
int main() {
  fprintf(stderr, "bench_sweep needs the CUDA build.\n");
  return 4;
}
#else
#include <cuda_runtime.h>

namespace {

struct Args {
  size_t min_bytes = 4096, max_bytes = size_t(1) << 30;
  std::vector<std::string> algos = {"auto"};
  bool symmetric = true, reg = false;
  std::string op = "allreduce";
};

[[noreturn]] void Usage(const std::string& why) {
  if (!why.empty()) fprintf(stderr, "bench_sweep: %s\n", why.c_str());
  fprintf(stderr,
          "usage: bench_sweep [--min BYTES] [--max BYTES] [--algos a,b,...] [--symmetric 0|1] [--register 0|1]\n"
          "                   [--op allreduce|reduce_scatter|all_gather]\n");
  exit(1);
}

Args Parse(int argc, char** argv) {
  Args a;
  for (int i = 1; i < argc; ++i) {
    const std::string s = argv[i];
    auto need = [&]() -> std::string {
      if (i + 1 >= argc) Usage(s + " needs a value");
      return argv[++i];
    };
    try {
      if (s == "--min") a.min_bytes = static_cast<size_t>(util::parse_number(need()));
      else if (s == "--max") a.max_bytes = static_cast<size_t>(util::parse_number(need()));
      else if (s == "--symmetric") a.symmetric = atoi(need().c_str()) != 0;
      else if (s == "--register") a.reg = atoi(need().c_str()) != 0;
      else if (s == "--op") a.op = need();
      else if (s == "--algos") {
        a.algos.clear();
        std::stringstream ss(need());
        std::string item;
        while (std::getline(ss, item, ',')) if (!item.empty()) a.algos.push_back(item);
      } else Usage("unknown option " + s);
    } catch (const util::MalformedNumber& e) {
      Usage(e.what());
    }
  }
  if (a.min_bytes < 4 || a.max_bytes < a.min_bytes) Usage("bad size range");
  if (a.op != "allreduce" && a.op != "reduce_scatter" && a.op != "all_gather") Usage("unknown --op " + a.op);
  if (a.algos.empty()) Usage("no algorithm");
  return a;
}

// Largest value over the ranks, through the host transport (values are sent
// as microsecond counts; SumOverRanks is the only reduction the bootstrap has).
double MaxOverRanks(ibcomm::Communicator* comm, int rank, int ws, double v) {
  double mx = v;
  for (int r = 0; r < ws; ++r) {
    const long long mine = (r == rank) ? static_cast<long long>(v * 1e6) : 0;
    const double got = static_cast<double>(ibcomm::SumOverRanks(comm, mine)) * 1e-6;
    mx = std::max(mx, got);
  }
  return mx;
}

}  // namespace

int main(int argc, char** argv) {
  const Args a = Parse(argc, argv);
  ibcomm::BootstrapEnv env = ibcomm::ReadBootstrapEnv();
  int ngpu = 0;
  CUDACHECK(cudaGetDeviceCount(&ngpu));
  if (ngpu < env.world_size)
    IBCOMM_FAIL(NOT_SUPPORTED, "%d ranks need %d GPUs, %d visible.\n", env.world_size, env.world_size, ngpu);
  CUDACHECK(cudaSetDevice(env.local_rank % ngpu));
  ibcomm::SetErrorPolicy(ibcomm::ErrorPolicy::kThrow);  // an algorithm that does not apply to a size is skipped

  ibcomm::Communicator comm(env.world_size);
  ibcomm::ConnectAll(&comm, env);
  const int ws = env.world_size, rank = env.rank;
  const size_t nmax = a.max_bytes / sizeof(float);
  float *in = nullptr, *out = nullptr;
  int reg_in = -1, reg_out = -1;
  if (a.symmetric && ws > 1) {
    in = static_cast<float*>(ibcomm::DeviceContextSymmetricAlloc(&comm, a.max_bytes));
    out = static_cast<float*>(ibcomm::DeviceContextSymmetricAlloc(&comm, a.max_bytes));
  } else {
    CUDACHECK(cudaMalloc(&in, a.max_bytes));
    CUDACHECK(cudaMalloc(&out, a.max_bytes));
    if (a.reg && ws > 1) {
      reg_in = comm.RegisterCudaBuffer(in, a.max_bytes);
      reg_out = comm.RegisterCudaBuffer(out, a.max_bytes);
    }
  }
  {
    std::vector<float> h(nmax);
    for (size_t i = 0; i < nmax; ++i) h[i] = static_cast<float>((i * 2654435761u >> 20) % 2001) - 1000.0f;
    CUDACHECK(cudaMemcpy(in, h.data(), nmax * sizeof(float), cudaMemcpyHostToDevice));
  }
  cudaStream_t stream;
  CUDACHECK(cudaStreamCreate(&stream));
  cudaEvent_t e0, e1;
  CUDACHECK(cudaEventCreate(&e0));
  CUDACHECK(cudaEventCreate(&e1));
  const bool rs = a.op == "reduce_scatter", ag = a.op == "all_gather";

  for (size_t bytes = a.min_bytes; bytes <= a.max_bytes; bytes *= 2) {
    size_t n = bytes / sizeof(float);
    if (rs || ag) n = n / static_cast<size_t>(ws) * static_cast<size_t>(ws);
    if (n < static_cast<size_t>(ws)) continue;
    const size_t block = n / static_cast<size_t>(ws);
    const int iters = bytes <= (size_t(1) << 20) ? 200 : (bytes <= (size_t(64) << 20) ? 50 : 10);
    const int warm = bytes <= (size_t(1) << 20) ? 20 : 5;
    for (const std::string& name : a.algos) {
      ibcomm::CudaAllreduceOptions o;
      o.stream = stream;
      o.use_stream = true;
      o.async = true;
      o.scale = ag ? 1.0 : 1.0 / ws;
      double ms = -1.0;
      std::string error;
      try {
        o.algo = ibcomm::AlgoFromName(name);
        auto call = [&] {
          if (rs) comm.ReduceScatterCuda(ibcomm::DType::kFloat32, in, out, block, o);
          else if (ag) comm.AllGatherCuda(ibcomm::DType::kFloat32, in, out, block, o);
          else comm.AllreduceCuda(ibcomm::DType::kFloat32, in, out, n, o);
        };
        for (int k = 0; k < warm; ++k) call();
        CUDACHECK(cudaStreamSynchronize(stream));
        ibcomm::DeviceContextCheck(comm.device());
        comm.Barrier();
        CUDACHECK(cudaEventRecord(e0, stream));
        for (int k = 0; k < iters; ++k) call();
        CUDACHECK(cudaEventRecord(e1, stream));
        CUDACHECK(cudaStreamSynchronize(stream));
        ibcomm::DeviceContextCheck(comm.device());
        float t = 0;
        CUDACHECK(cudaEventElapsedTime(&t, e0, e1));
        ms = static_cast<double>(t) / iters;
      } catch (const ibcomm::Error& e) {
        error = e.what();
      }
      // Every rank takes part in the reduction, whether its call worked or not.
      const double worst = MaxOverRanks(&comm, rank, ws, ms < 0 ? 0.0 : ms);
      const long long failed = ibcomm::SumOverRanks(&comm, ms < 0 ? 1 : 0);
      if (rank != 0) continue;
      if (failed != 0) {
        for (char& c : error)
          if (c == '"' || c == '\n') c = ' ';
        printf("{\"op\": \"%s\", \"bytes\": %zu, \"algo\": \"%s\", \"error\": \"%s\"}\n", a.op.c_str(), n * sizeof(float),
               name.c_str(), error.c_str());
        continue;
      }
      const ibcomm::DeviceInfo info = ibcomm::DeviceContextInfo(comm.device());
      const double factor = ws > 1 ? ((rs || ag) ? static_cast<double>(ws - 1) / ws : 2.0 * (ws - 1) / ws) : 1.0;
      const double algbw = static_cast<double>(n * sizeof(float)) / (worst * 1e-3) / 1e9;
      printf("{\"op\": \"%s\", \"bytes\": %zu, \"algo\": \"%s\", \"chosen\": \"%s\", \"channels\": %d, \"us\": %.2f, "
             "\"algbw_gbs\": %.1f, \"busbw_gbs\": %.1f, \"n_gpus\": %d, \"buffers\": \"%s\"}\n",
             a.op.c_str(), n * sizeof(float), name.c_str(), ibcomm::AlgoName(static_cast<ibcomm::Algo>(info.last_algo)),
             info.last_channels, worst * 1e3, algbw, algbw * factor, ws,
             a.symmetric && ws > 1 ? "symmetric" : (reg_in >= 0 && reg_out >= 0 ? "registered" : "plain"));
      fflush(stdout);
    }
  }
  comm.Barrier();
  if (reg_in >= 0) comm.DeregisterCudaBuffer(reg_in);
  if (reg_out >= 0) comm.DeregisterCudaBuffer(reg_out);
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  cudaStreamDestroy(stream);
  if (a.symmetric && ws > 1) {
    ibcomm::DeviceContextSymmetricFree(&comm, in);
    ibcomm::DeviceContextSymmetricFree(&comm, out);
  } else {
    cudaFree(in);
    cudaFree(out);
  }
  return 0;
}
#endif
