// Local streaming kernel: out[i] = cast(in[i] * scale).
//
// Used for world_size == 1 (the reference's whole-buffer cudaMemcpy,
// ibcomm/allreduce_cuda_impl.h:40-46, 332-340, with the scale and the type
// conversion fused in) and for local staging copies.  Tiles travel
// global -> shared -> global with the bulk asynchronous copy engine (TMA,
// non-tensor form `cp.async.bulk`, no cluster multicast): one elected thread
// issues the copies and an mbarrier reports their arrival, the CTA's threads
// only touch shared memory.  A multi-stage ring of tiles keeps loads, math and
// stores of different tiles in flight at once.  Every wait is bounded.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "ibcomm/communicator.h"
#include "kernels.h"
#include "vec_ops.cuh"

namespace ibcomm {
namespace dev {

constexpr int kCopyThreads = 256;
constexpr int kCopyStages = 4;
constexpr int kCopyTileBytesIn = 16384;  // bytes of input per tile
constexpr uint32_t kMbarSpinLimit = 1u << 22;

__device__ __forceinline__ uint32_t SmemAddr(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void MbarInit(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(SmemAddr(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void MbarExpectTx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(SmemAddr(bar)), "r"(bytes) : "memory");
}
// Bounded wait on a phase; false when the limit ran out.
__device__ __forceinline__ bool MbarWait(uint64_t* bar, uint32_t parity) {
  for (uint32_t spin = 0; spin < kMbarSpinLimit; ++spin) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(SmemAddr(bar)), "r"(parity)
        : "memory");
    if (done) return true;
  }
  return false;
}
__device__ __forceinline__ void BulkLoad(void* smem_dst, const void* gmem_src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(SmemAddr(smem_dst)),
               "l"(gmem_src), "r"(bytes), "r"(SmemAddr(bar))
               : "memory");
}
__device__ __forceinline__ void BulkStore(void* gmem_dst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gmem_dst), "r"(SmemAddr(smem_src)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void BulkCommit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void BulkWaitRead() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void BulkWaitAll() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void FenceProxyAsync() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// Tiles of `kTileElems` elements.  Requires 16-byte aligned `in` and `out`;
// the ragged end (less than one 16-byte vector of either type) is finished
// with plain loads and stores.
template <typename TI, typename TO>
__global__ void __launch_bounds__(kCopyThreads) CopyScaleTmaKernel(const TI* __restrict__ in, TO* __restrict__ out, uint64_t n,
                                                                   double scale, uint32_t* doorbell) {
  using A = typename Acc<TI>::type;
  constexpr int kTileElems = kCopyTileBytesIn / static_cast<int>(sizeof(TI));
  constexpr int kOutTileBytes = kTileElems * static_cast<int>(sizeof(TO));
  extern __shared__ __align__(128) unsigned char smem[];
  TI* in_tiles = reinterpret_cast<TI*>(smem);
  TO* out_tiles = reinterpret_cast<TO*>(smem + kCopyStages * kCopyTileBytesIn);
  __shared__ uint64_t full_bar[kCopyStages];
  __shared__ int s_fail;

  // Elements that can move as whole 16-byte vectors in both types.
  constexpr uint64_t kQuantum = 16 / (sizeof(TI) < sizeof(TO) ? sizeof(TI) : sizeof(TO));
  const uint64_t n_bulk = n / kQuantum * kQuantum;
  const uint64_t num_tiles = (n_bulk + kTileElems - 1) / kTileElems;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kCopyStages; ++s) MbarInit(&full_bar[s], 1);
    s_fail = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  auto tile_elems = [&](uint64_t t) -> uint32_t {
    const uint64_t b = t * kTileElems;
    const uint64_t e = b + kTileElems < n_bulk ? b + kTileElems : n_bulk;
    return static_cast<uint32_t>(e - b);
  };

  // This CTA's tiles: blockIdx.x, blockIdx.x + gridDim.x, ...
  const uint64_t first = blockIdx.x, step = gridDim.x;
  const uint64_t my_tiles = first < num_tiles ? (num_tiles - first + step - 1) / step : 0;

  if (threadIdx.x == 0) {
    for (uint64_t k = 0; k < my_tiles && k < kCopyStages; ++k) {
      const uint64_t t = first + k * step;
      const uint32_t bytes = tile_elems(t) * static_cast<uint32_t>(sizeof(TI));
      MbarExpectTx(&full_bar[k], bytes);
      BulkLoad(in_tiles + k * kTileElems, in + t * kTileElems, bytes, &full_bar[k]);
    }
  }

  for (uint64_t k = 0; k < my_tiles; ++k) {
    const int s = static_cast<int>(k % kCopyStages);
    const uint32_t parity = static_cast<uint32_t>((k / kCopyStages) & 1);
    const uint64_t t = first + k * step;
    const uint32_t cnt = tile_elems(t);
    if (!MbarWait(&full_bar[s], parity)) s_fail = 1;
    // The store that last read out_tiles[s] (tile k - kCopyStages) must be done
    // reading shared memory before the slot is overwritten.
    if (threadIdx.x == 0) BulkWaitRead<kCopyStages - 1>();
    __syncthreads();
    if (s_fail) break;
    const TI* src = in_tiles + s * kTileElems;
    TO* dst = out_tiles + s * kTileElems;
    for (uint32_t i = threadIdx.x; i < cnt; i += kCopyThreads) {
      A v = ToAcc<A, TI>(src[i]);
      dst[i] = FromAcc<TO, A>(ScaleAcc<A>(v, scale));
    }
    FenceProxyAsync();
    __syncthreads();
    if (threadIdx.x == 0) {
      BulkStore(out + t * kTileElems, dst, cnt * static_cast<uint32_t>(sizeof(TO)));
      BulkCommit();
      const uint64_t kn = k + kCopyStages;
      if (kn < my_tiles) {
        const uint64_t tn = first + kn * step;
        const uint32_t bytes = tile_elems(tn) * static_cast<uint32_t>(sizeof(TI));
        MbarExpectTx(&full_bar[s], bytes);
        BulkLoad(in_tiles + s * kTileElems, in + tn * kTileElems, bytes, &full_bar[s]);
      }
    }
  }
  if (threadIdx.x == 0) {
    BulkWaitAll();
    if (s_fail && doorbell != nullptr) *reinterpret_cast<volatile uint32_t*>(doorbell) = kStatusWaitTimeout;
  }
  // Ragged end.
  if (blockIdx.x == 0) {
    for (uint64_t i = n_bulk + threadIdx.x; i < n; i += kCopyThreads) {
      A v = ToAcc<A, TI>(in[i]);
      out[i] = FromAcc<TO, A>(ScaleAcc<A>(v, scale));
    }
  }
  (void)kOutTileBytes;
}

// Plain grid-stride variant for unaligned buffers.
template <typename TI, typename TO>
__global__ void __launch_bounds__(kCopyThreads) CopyScaleSimpleKernel(const TI* __restrict__ in, TO* __restrict__ out, uint64_t n, double scale) {
  using A = typename Acc<TI>::type;
  for (uint64_t i = blockIdx.x * static_cast<uint64_t>(kCopyThreads) + threadIdx.x; i < n; i += static_cast<uint64_t>(gridDim.x) * kCopyThreads) {
    A v = ToAcc<A, TI>(in[i]);
    out[i] = FromAcc<TO, A>(ScaleAcc<A>(v, scale));
  }
}

}  // namespace dev

template <typename TI, typename TO>
static cudaError_t LaunchCopyTyped(const CopyParams& p, int blocks, cudaStream_t stream, uint32_t* doorbell) {
  const TI* in = static_cast<const TI*>(p.in);
  TO* out = static_cast<TO*>(p.out);
  if (p.len_elements == 0) return cudaSuccess;
  const bool aligned = ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out)) & 15u) == 0;
  if (!aligned) {
    dev::CopyScaleSimpleKernel<TI, TO><<<blocks, dev::kCopyThreads, 0, stream>>>(in, out, p.len_elements, p.scale);
    return cudaGetLastError();
  }
  constexpr int kTileElems = dev::kCopyTileBytesIn / static_cast<int>(sizeof(TI));
  const size_t smem = static_cast<size_t>(dev::kCopyStages) * (dev::kCopyTileBytesIn + kTileElems * sizeof(TO));
  static thread_local bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(dev::CopyScaleTmaKernel<TI, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return e;
    configured = true;
  }
  const uint64_t tiles = (p.len_elements + kTileElems - 1) / kTileElems;
  if (static_cast<uint64_t>(blocks) > tiles) blocks = static_cast<int>(tiles);
  if (blocks < 1) blocks = 1;
  dev::CopyScaleTmaKernel<TI, TO><<<blocks, dev::kCopyThreads, smem, stream>>>(in, out, p.len_elements, p.scale, doorbell);
  return cudaGetLastError();
}

cudaError_t LaunchCopyKernelWithDoorbell(const CopyParams& p, int blocks, cudaStream_t stream, uint32_t* doorbell) {
  const DType ti = static_cast<DType>(p.dtype_in), to = static_cast<DType>(p.dtype_out);
  if (ti == DType::kFloat32 && to == DType::kFloat32) return LaunchCopyTyped<float, float>(p, blocks, stream, doorbell);
  if (ti == DType::kFloat32 && to == DType::kBFloat16) return LaunchCopyTyped<float, __nv_bfloat16>(p, blocks, stream, doorbell);
  if (ti == DType::kFloat32 && to == DType::kFloat16) return LaunchCopyTyped<float, __half>(p, blocks, stream, doorbell);
  if (ti == DType::kBFloat16 && to == DType::kFloat32) return LaunchCopyTyped<__nv_bfloat16, float>(p, blocks, stream, doorbell);
  if (ti == DType::kFloat16 && to == DType::kFloat32) return LaunchCopyTyped<__half, float>(p, blocks, stream, doorbell);
  if (ti == DType::kFloat64 && to == ti) return LaunchCopyTyped<double, double>(p, blocks, stream, doorbell);
  if (ti == DType::kInt32 && to == ti) return LaunchCopyTyped<int, int>(p, blocks, stream, doorbell);
  if (ti == DType::kInt64 && to == ti) return LaunchCopyTyped<long long, long long>(p, blocks, stream, doorbell);
  if (ti == DType::kFloat16 && to == ti) return LaunchCopyTyped<__half, __half>(p, blocks, stream, doorbell);
  if (ti == DType::kBFloat16 && to == ti) return LaunchCopyTyped<__nv_bfloat16, __nv_bfloat16>(p, blocks, stream, doorbell);
  return cudaErrorInvalidValue;
}

cudaError_t LaunchCopyKernel(const CopyParams& p, int blocks, cudaStream_t stream) {
  return LaunchCopyKernelWithDoorbell(p, blocks, stream, nullptr);
}

}  // namespace ibcomm
