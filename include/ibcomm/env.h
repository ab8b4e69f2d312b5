// Environment knobs.  Names, defaults, validation and exit codes follow the
// reference (ibverbs_communicator.cpp:619-635, memory_pool.h:139-173,
// ibverbs_communicator_cuda.cpp:12-22); their meaning on an NVLink box:
//
//   IBCOMM_CHUNKSIZE              bytes per flag-synchronised pipeline unit
//   IBCOMM_MEMORY_POOL_PRE_ALLOC  bytes of the peer-mapped staging pool
//   IBCOMM_WORK_GPU_MEMORY_SIZE   bytes of the Rabenseifner landing region
//   IBCOMM_NUM_CUDA_STREAM        number of channels (CTAs) a call may use
//
// Values are read with atoi semantics ("1k" is 1), like the reference.
#pragma once

#include <cstddef>
#include <cstdint>
#include <string>

namespace ibcomm {
namespace env {

constexpr int kDefaultNumCudaStream = 256;
constexpr size_t kDefaultPoolPreAlloc = 64ull << 20;
constexpr size_t kDefaultWorkGpuMemory = 32ull << 20;
constexpr int kDefaultTimeoutMs = 10000;

// > 0 when set, 0 when unset.  <= 0 while set is INVALID_ARGUMENT (exit 1).
int64_t ReadChunkSize();
// 1..1024, default 256 (the reference's code says 128, memory_pool.h:82, its
// README 64; here the value caps the CTAs of a collective, and the ring and
// Rabenseifner kernels measure best with two 256-thread CTAs per SM).
// Outside the range is INVALID_ARGUMENT.
int ReadNumCudaStream();
// 4..1 GiB, default 64 MiB.  Outside the range is INVALID_ARGUMENT.
size_t ReadPreAllocSize();
// Default 32 MiB; non-positive values fall back to the default with a warning.
size_t ReadWorkGpuMemorySize();
// Trace file prefix, default "ibcomm_trace".
std::string ReadTraceFile();
// Device-side and host-side wait limit in milliseconds, default 10 s.
int ReadTimeoutMs();
// auto | ring | rabenseifner | nvls | oneshot | direct ; default auto.
std::string ReadAlgo();
bool ReadDisableNvls();
std::string ReadTuningFile();

}  // namespace env
}  // namespace ibcomm
