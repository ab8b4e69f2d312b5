// One-shot allreduce of several ranks on one GPU with its scratch memory in a
// file-scope device array: the entry point described in ibcomm/no_alloc.h,
// for callers that may not allocate.  It has no counterpart in the reference.
#include "ibcomm/no_alloc.h"

#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <mutex>

namespace {

constexpr int kMaxRanks = IBCOMM_NO_ALLOC_MAX_RANKS;
constexpr int kMaxCtas = 4;  // CTAs per rank
constexpr int kThreads = 256;
constexpr size_t kSlotBytes = IBCOMM_NO_ALLOC_MAX_BYTES;
constexpr int kMaxDevices = 64;

// Layout of the scratch array.
struct Scratch {
  // flag[parity][owner][cta][source]: call number of the last delivery.
  unsigned long long flag[2][kMaxRanks][kMaxCtas][kMaxRanks];
  unsigned int error;  // non-zero when a wait ran out
  unsigned int pad_[63];
  // slot[parity][owner][source]: the source rank's message as the owner sees it.
  unsigned char slot[2][kMaxRanks][kMaxRanks][kSlotBytes];
};

// Lives in the library image on every device that loads it.  In host code this
// name is only a stand-in; the device address comes from cudaGetSymbolAddress.
static __device__ __align__(256) unsigned char g_scratch[sizeof(Scratch)];

struct Params {
  const float* send[kMaxRanks];
  float* recv[kMaxRanks];
  Scratch* scratch;
  unsigned long long seq;
  unsigned long long timeout_ns;
  unsigned long long n;
  float scale;
  int ws;
  int parity;
};

__device__ __forceinline__ unsigned long long LdAcquire(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void StRelease(unsigned long long* p, unsigned long long v) {
  asm volatile("st.release.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long TimerNs() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// grid = (ctas, ranks); launched cooperatively, because the CTAs of different
// ranks wait for each other.
__global__ void __launch_bounds__(kThreads) OneShotNoAllocKernel(const __grid_constant__ Params p) {
  const int cta = blockIdx.x, ncta = gridDim.x, me = blockIdx.y, ws = p.ws;
  Scratch* s = p.scratch;
  __shared__ int s_stop;
  if (threadIdx.x == 0) s_stop = 0;
  __syncthreads();
  // This CTA's element range, a multiple of 4 elements so that 16-byte vectors can be used.
  const unsigned long long nvec = (p.n + 3) / 4;
  const unsigned long long per = (nvec + ncta - 1) / ncta;
  unsigned long long lo = per * cta * 4, hi = lo + per * 4;
  if (lo > p.n) lo = p.n;
  if (hi > p.n) hi = p.n;
  const float* mine = p.send[me];
  float* out = p.recv[me];
  const bool vec_ok = ((reinterpret_cast<uintptr_t>(mine) | reinterpret_cast<uintptr_t>(out)) & 15u) == 0;
  const unsigned long long nfull = vec_ok ? (hi - lo) / 4 : 0;

  // (1) my slice into every other rank's slot for me.
  for (int k = 1; k < ws; ++k) {
    const int q = (me + k) % ws;
    float* dst = reinterpret_cast<float*>(s->slot[p.parity][q][me]);
    for (unsigned long long i = threadIdx.x; i < nfull; i += blockDim.x)
      reinterpret_cast<float4*>(dst + lo)[i] = reinterpret_cast<const float4*>(mine + lo)[i];
    for (unsigned long long i = lo + nfull * 4 + threadIdx.x; i < hi; i += blockDim.x) dst[i] = mine[i];
  }
  __syncthreads();
  // (2) raise my flag at every other rank, (3) wait for theirs (bounded).
  if (threadIdx.x < ws && static_cast<int>(threadIdx.x) != me) {
    const int q = threadIdx.x;
    __threadfence();
    StRelease(&s->flag[p.parity][q][cta][me], p.seq);
    const unsigned long long* f = &s->flag[p.parity][me][cta][q];
    const unsigned long long t0 = TimerNs();
    unsigned spin = 0;
    while (LdAcquire(f) < p.seq) {
      if ((++spin & 63u) == 0) {
        if (*reinterpret_cast<volatile unsigned int*>(&s->error) != 0 || TimerNs() - t0 > p.timeout_ns) {
          s->error = 1;
          __threadfence();
          s_stop = 1;
          break;
        }
      }
    }
  }
  __syncthreads();
  if (s_stop) return;
  // (4) add the copies in rank order.
  for (unsigned long long i = threadIdx.x; i < nfull; i += blockDim.x) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int q = 0; q < ws; ++q) {
      const float* src = (q == me) ? mine : reinterpret_cast<const float*>(s->slot[p.parity][me][q]);
      const float4 v = __ldcv(reinterpret_cast<const float4*>(src + lo) + i);
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    if (p.scale != 1.0f) { acc.x *= p.scale; acc.y *= p.scale; acc.z *= p.scale; acc.w *= p.scale; }
    reinterpret_cast<float4*>(out + lo)[i] = acc;
  }
  for (unsigned long long i = lo + nfull * 4 + threadIdx.x; i < hi; i += blockDim.x) {
    float acc = 0.f;
    for (int q = 0; q < ws; ++q) {
      const float* src = (q == me) ? mine : reinterpret_cast<const float*>(s->slot[p.parity][me][q]);
      acc += __ldcv(src + i);
    }
    if (p.scale != 1.0f) acc *= p.scale;
    out[i] = acc;
  }
}

void Describe(char* errbuf, size_t len, const char* fmt, ...) {
  if (errbuf == nullptr || len == 0) return;
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(errbuf, len, fmt, ap);
  va_end(ap);
}

// Per-device state kept on the host: the scratch address and the call count.
struct DeviceState {
  Scratch* scratch = nullptr;
  unsigned long long calls = 0;
};
DeviceState g_state[kMaxDevices];
std::mutex g_mutex;

}  // namespace

extern "C" int ibcomm_emu_oneshot_allreduce_f32_noalloc(const float* const* sendbufs, float* const* recvbufs,
                                                         int num_ranks, size_t len_elements, float scale, void* stream_v,
                                                         char* errbuf, size_t errbuf_len) {
  if (errbuf != nullptr && errbuf_len > 0) errbuf[0] = '\0';
  if (sendbufs == nullptr || recvbufs == nullptr) {
    Describe(errbuf, errbuf_len, "sendbufs and recvbufs must not be null");
    return 1;
  }
  if (num_ranks < 1 || num_ranks > kMaxRanks) {
    Describe(errbuf, errbuf_len, "num_ranks = %d is outside 1..%d", num_ranks, kMaxRanks);
    return 1;
  }
  // Compared in elements: `len_elements * sizeof(float)` wraps for absurd lengths.
  if (len_elements > kSlotBytes / sizeof(float)) {
    Describe(errbuf, errbuf_len, "%zu elements = %zu bytes per buffer exceed the limit of %zu bytes of the no-allocation entry point",
             len_elements, len_elements <= (~size_t(0)) / sizeof(float) ? len_elements * sizeof(float) : ~size_t(0), kSlotBytes);
    return 1;
  }
  for (int r = 0; r < num_ranks; ++r) {
    if (sendbufs[r] == nullptr || recvbufs[r] == nullptr) {
      Describe(errbuf, errbuf_len, "buffer of rank %d is null", r);
      return 1;
    }
  }
  if (len_elements == 0) return 0;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    Describe(errbuf, errbuf_len, "cudaGetDevice failed: %s", cudaGetErrorString(e));
    return 3;
  }
  std::lock_guard<std::mutex> lock(g_mutex);
  DeviceState& st = g_state[dev];
  if (st.scratch == nullptr) {
    // Once per device, with that device current: the device address of the array.
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_scratch);
    if (e != cudaSuccess || ptr == nullptr) {
      Describe(errbuf, errbuf_len, "cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
      return 3;
    }
    st.scratch = static_cast<Scratch*>(ptr);
  }
  Params p;
  for (int r = 0; r < kMaxRanks; ++r) {
    p.send[r] = r < num_ranks ? sendbufs[r] : nullptr;
    p.recv[r] = r < num_ranks ? recvbufs[r] : nullptr;
  }
  p.scratch = st.scratch;
  p.seq = ++st.calls;
  p.parity = static_cast<int>(p.seq & 1u);
  p.timeout_ns = 2000000000ull;
  p.n = len_elements;
  p.scale = scale;
  p.ws = num_ranks;
  // The error word must start at zero; the flags only grow and need no clearing.
  e = cudaMemsetAsync(&st.scratch->error, 0, sizeof(unsigned int), stream);
  if (e != cudaSuccess) {
    Describe(errbuf, errbuf_len, "cudaMemsetAsync failed: %s", cudaGetErrorString(e));
    return 3;
  }
  int ctas = static_cast<int>((len_elements * sizeof(float) + 8191) / 8192);
  if (ctas > kMaxCtas) ctas = kMaxCtas;
  if (ctas < 1) ctas = 1;
  dim3 grid(static_cast<unsigned>(ctas), static_cast<unsigned>(num_ranks));
  void* args[] = {&p};
  e = cudaLaunchCooperativeKernel(reinterpret_cast<void*>(OneShotNoAllocKernel), grid, dim3(kThreads), args, 0, stream);
  if (e != cudaSuccess) {
    Describe(errbuf, errbuf_len, "kernel launch failed: %s", cudaGetErrorString(e));
    return 3;
  }
  unsigned int err = 0;
  e = cudaMemcpyAsync(&err, &st.scratch->error, sizeof(err), cudaMemcpyDeviceToHost, stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
  if (e != cudaSuccess) {
    Describe(errbuf, errbuf_len, "waiting for the kernel failed: %s", cudaGetErrorString(e));
    return 3;
  }
  if (err != 0) {
    Describe(errbuf, errbuf_len, "a wait inside the kernel ran out after %llu ms", p.timeout_ns / 1000000ull);
    return 2;
  }
  return 0;
}
