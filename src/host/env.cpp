#include "ibcomm/env.h"

#include <cstdlib>
#include <cstring>

#include "ibcomm/error.h"

namespace ibcomm {
namespace env {

int64_t ReadChunkSize() {
  const char* s = getenv("IBCOMM_CHUNKSIZE");
  if (s == nullptr) return 0;
  int v = atoi(s);
  if (v <= 0)
    IBCOMM_FAIL(INVALID_ARGUMENT, "IBCOMM_CHUNKSIZE must be a positive integer (got '%s').\n", s);
  return v;
}

int ReadNumCudaStream() {
  const char* s = getenv("IBCOMM_NUM_CUDA_STREAM");
  if (s == nullptr) return kDefaultNumCudaStream;
  int v = atoi(s);
  if (v < 1 || v > 1024)
    IBCOMM_FAIL(INVALID_ARGUMENT, "IBCOMM_NUM_CUDA_STREAM must be in 1..1024 (got '%s').\n", s);
  return v;
}

size_t ReadPreAllocSize() {
  const char* s = getenv("IBCOMM_MEMORY_POOL_PRE_ALLOC");
  if (s == nullptr) return kDefaultPoolPreAlloc;
  long long v = atoll(s);
  if (v < 4 || v > (1ll << 30))
    IBCOMM_FAIL(INVALID_ARGUMENT,
                "IBCOMM_MEMORY_POOL_PRE_ALLOC must be in 4..1073741824 bytes (got '%s').\n", s);
  return static_cast<size_t>(v);
}

size_t ReadWorkGpuMemorySize() {
  const char* s = getenv("IBCOMM_WORK_GPU_MEMORY_SIZE");
  if (s == nullptr) return kDefaultWorkGpuMemory;
  long long v = atoll(s);
  if (v <= 0) {
    IBCOMM_WARN("IBCOMM_WORK_GPU_MEMORY_SIZE='%s' is not a positive size; using %zu bytes.\n", s,
                kDefaultWorkGpuMemory);
    return kDefaultWorkGpuMemory;
  }
  return static_cast<size_t>(v);
}

std::string ReadTraceFile() {
  const char* s = getenv("IBCOMM_TRACE_FILE");
  return s ? std::string(s) : std::string("ibcomm_trace");
}

int ReadTimeoutMs() {
  const char* s = getenv("IBCOMM_TIMEOUT_MS");
  if (s == nullptr) return kDefaultTimeoutMs;
  int v = atoi(s);
  return v > 0 ? v : kDefaultTimeoutMs;
}

std::string ReadAlgo() {
  const char* s = getenv("IBCOMM_ALGO");
  return s ? std::string(s) : std::string("auto");
}

bool ReadDisableNvls() {
  const char* s = getenv("IBCOMM_DISABLE_NVLS");
  return s != nullptr && s[0] != '\0' && strcmp(s, "0") != 0;
}

std::string ReadTuningFile() {
  const char* s = getenv("IBCOMM_TUNING_FILE");
  return s ? std::string(s) : std::string();
}

}  // namespace env
}  // namespace ibcomm
