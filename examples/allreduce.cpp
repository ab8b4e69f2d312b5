// Example and acceptance test: allreduce of one large fp32 buffer, timed, with
// the result checked on every rank — the program the reference ships as
// examples/allreduce.cpp (256 MiB buffer, three warm-up runs, the time of the
// last run is reported, every rank prints OK or FAIL).
//
//   ibcomm_run -np 8 build/bin/allreduce_cuda            # device buffers, ring kernel
//   ibcomm_run -np 4 build/bin/allreduce rabenseifner    # host buffers
//   ... [ring|rabenseifner|auto|nvls|oneshot] [elements]
//
// Built without -DUSE_CUDA the buffers live on the host and travel over the
// shared-memory transport; with it they live on the GPU selected by the
// local rank.  The ranks are started by ibcomm_run (no MPI); the expected
// values are known in closed form because every rank fills its buffer from
// the same seeded generator.
#include <time.h>

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <random>
#include <string>
#include <vector>

#include "ibcomm/bootstrap.h"
#include "ibcomm/communicator.h"

#ifdef USE_CUDA
#include <cuda_runtime.h>
#endif

namespace {
constexpr size_t kArrayLength = 67108864;  // 256 MiB of float
constexpr int kWarmup = 3;

double Now() {
  struct timespec ts;
  clock_gettime(CLOCK_MONOTONIC_RAW, &ts);
  return static_cast<double>(ts.tv_sec) + static_cast<double>(ts.tv_nsec) * 1e-9;
}
}  // namespace

int main(int argc, char** argv) {
  const std::string algo = argc > 1 ? argv[1] : "ring";
  const size_t n = argc > 2 ? static_cast<size_t>(util::parse_number(argv[2])) : kArrayLength;
  ibcomm::BootstrapEnv env = ibcomm::ReadBootstrapEnv();

#ifdef USE_CUDA
  int ngpu = 0;
  CUDACHECK(cudaGetDeviceCount(&ngpu));
  if (ngpu < env.world_size)
    IBCOMM_FAIL(NOT_SUPPORTED, "%d ranks need %d GPUs, %d visible.\n", env.world_size, env.world_size, ngpu);
  CUDACHECK(cudaSetDevice(env.local_rank % ngpu));
#endif

  ibcomm::Communicator comm(env.world_size);
  ibcomm::ConnectAll(&comm, env);

  // Integer-valued floats in [-1000, 1000], identical on every rank: the sum
  // over N ranks is exactly N times the value.
  std::vector<float> host_in(n), host_out(n, 0.0f);
  std::mt19937 gen(0);
  std::uniform_int_distribution<int> dist(-1000, 1000);
  for (size_t i = 0; i < n; ++i) host_in[i] = static_cast<float>(dist(gen));

#ifdef USE_CUDA
  float *d_in = nullptr, *d_out = nullptr;
  CUDACHECK(cudaMalloc(&d_in, n * sizeof(float)));
  CUDACHECK(cudaMalloc(&d_out, n * sizeof(float)));
  CUDACHECK(cudaMemcpy(d_in, host_in.data(), n * sizeof(float), cudaMemcpyHostToDevice));
  auto run = [&] {
    if (algo == "ring") {
      comm.AllreduceRingCuda(d_in, d_out, n);
    } else if (algo == "rabenseifner") {
      comm.AllreduceRabenseifnerCuda(d_in, d_out, n);
    } else {
      ibcomm::CudaAllreduceOptions o;
      o.algo = ibcomm::AlgoFromName(algo);
      comm.AllreduceCuda(ibcomm::DType::kFloat32, d_in, d_out, n, o);
    }
  };
#else
  auto run = [&] {
    if (algo == "rabenseifner") comm.AllreduceRabenseifner(host_in.data(), host_out.data(), n);
    else comm.AllreduceRing(host_in.data(), host_out.data(), n);
  };
#endif

  comm.SetTimerBase();
  double elapsed = 0;
  for (int it = 0; it < kWarmup + 1; ++it) {
    comm.Barrier();
    const double t0 = Now();
    run();
    elapsed = Now() - t0;
  }

#ifdef USE_CUDA
  CUDACHECK(cudaMemcpy(host_out.data(), d_out, n * sizeof(float), cudaMemcpyDeviceToHost));
  CUDACHECK(cudaFree(d_in));
  CUDACHECK(cudaFree(d_out));
#endif

  bool ok = true;
  size_t reported = 0;
  for (size_t i = 0; i < n; ++i) {
    const float want = host_in[i] * static_cast<float>(env.world_size);
    if (std::fabs(host_out[i] - want) > 1e-6f) {
      ok = false;
      if (reported++ < 10) fprintf(stderr, "rank %d: element %zu is %f, expected %f\n", env.rank, i, host_out[i], want);
    }
  }
  for (int r = 0; r < env.world_size; ++r) {
    if (r == env.rank) printf("rank: %d %s\n", env.rank, ok ? "OK" : "FAIL");
    fflush(stdout);
    comm.Barrier();
  }
  const long long failed = ibcomm::SumOverRanks(&comm, ok ? 0 : 1);
  if (env.rank == 0) {
    printf("elapsed time : %e [s]\n", elapsed);
    const double bytes = static_cast<double>(n) * sizeof(float);
    const int ws = env.world_size;
    printf("algorithm bandwidth : %.3f GB/s, bus bandwidth : %.3f GB/s\n", bytes / elapsed / 1e9,
           ws > 1 ? bytes / elapsed / 1e9 * 2.0 * (ws - 1) / ws : bytes / elapsed / 1e9);
  }
  return failed == 0 ? 0 : 1;
}
