// Local streaming kernel: out[i] = cast(in[i] * scale).
//
// Used for world_size == 1 (the reference's whole-buffer cudaMemcpy,
// ibcomm/allreduce_cuda_impl.h:40-46, 332-340, with the scale and the type
// conversion fused in) and for local staging copies.  Input tiles travel
// global -> shared with the bulk asynchronous copy engine (TMA, non-tensor
// form `cp.async.bulk`, no cluster multicast).  Every warp runs its own
// pipeline: a ring of four 4 KiB tiles with one mbarrier each, refilled by the
// warp's first lane, so 128 KiB of loads are in flight per SM without
// occupying registers and no CTA-wide barrier sits on the critical path.  The
// lanes read a tile from shared memory, scale and convert it, and write the
// result with 16-byte global stores.  Every wait is bounded.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cstdlib>

#include "ibcomm/communicator.h"
#include "kernels.h"
#include "tma_stage.cuh"
#include "vec_ops.cuh"

namespace ibcomm {
namespace dev {

#ifndef IBCOMM_COPY_THREADS
#define IBCOMM_COPY_THREADS 256
#endif
constexpr int kCopyThreads = IBCOMM_COPY_THREADS;
constexpr int kCopyWarps = kCopyThreads / 32;
#ifndef IBCOMM_COPY_STAGES
#define IBCOMM_COPY_STAGES 4
#endif
#ifndef IBCOMM_COPY_TILE
#define IBCOMM_COPY_TILE 4096
#endif
constexpr int kCopyStages = IBCOMM_COPY_STAGES;      // tiles in flight per warp
constexpr int kCopyTileBytesIn = IBCOMM_COPY_TILE;   // bytes of input per tile
// Tiles of `kTileElems` elements, dealt round-robin to the warps of the grid.
// Requires 16-byte aligned `in` and `out`; the ragged end (less than one
// 16-byte vector of either type) is finished with plain loads and stores.
template <typename TI, typename TO>
__global__ void __launch_bounds__(kCopyThreads) CopyScaleTmaKernel(const TI* __restrict__ in, TO* __restrict__ out, uint64_t n,
                                                                   double scale, uint32_t* doorbell) {
  using A = typename Acc<TI>::type;
  constexpr int kTileElems = kCopyTileBytesIn / static_cast<int>(sizeof(TI));
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ uint64_t full_bar[kCopyWarps][kCopyStages];
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  TI* my_tiles_smem = reinterpret_cast<TI*>(smem + static_cast<size_t>(warp) * kCopyStages * kCopyTileBytesIn);

  // Elements that move as whole 16-byte vectors in both types.
  constexpr int kQ = 16 / static_cast<int>(sizeof(TI) < sizeof(TO) ? sizeof(TI) : sizeof(TO));
  constexpr int kNI = kQ / VecIO<TI>::kN;  // input vectors per quantum
  constexpr int kNO = kQ / VecIO<TO>::kN;  // output vectors per quantum
  const uint64_t n_bulk = n / kQ * kQ;
  const uint64_t num_tiles = (n_bulk + kTileElems - 1) / kTileElems;
  const bool do_scale = scale != 1.0;

  if (lane == 0) {
    for (int s = 0; s < kCopyStages; ++s) MbarInit(&full_bar[warp][s], 1);
    MbarInitFence();
  }
  __syncwarp();

  auto tile_elems = [&](uint64_t t) -> uint32_t {
    const uint64_t b = t * kTileElems;
    const uint64_t e = b + kTileElems < n_bulk ? b + kTileElems : n_bulk;
    return static_cast<uint32_t>(e - b);
  };

  // This warp's tiles: first, first + step, ...
  const uint64_t first = static_cast<uint64_t>(blockIdx.x) * kCopyWarps + warp;
  const uint64_t step = static_cast<uint64_t>(gridDim.x) * kCopyWarps;
  const uint64_t my_tiles = first < num_tiles ? (num_tiles - first + step - 1) / step : 0;

  if (lane == 0) {
    for (uint64_t k = 0; k < my_tiles && k < kCopyStages; ++k) {
      const uint64_t t = first + k * step;
      const uint32_t bytes = tile_elems(t) * static_cast<uint32_t>(sizeof(TI));
      MbarExpectTx(&full_bar[warp][k], bytes);
      BulkLoad(my_tiles_smem + k * kTileElems, in + t * kTileElems, bytes, &full_bar[warp][k]);
    }
  }
  __syncwarp();

  bool failed = false;
  for (uint64_t k = 0; k < my_tiles; ++k) {
    const int s = static_cast<int>(k % kCopyStages);
    const uint32_t parity = static_cast<uint32_t>((k / kCopyStages) & 1);
    const uint64_t t = first + k * step;
    const uint32_t quanta = tile_elems(t) / kQ;
    if (!MbarWait(&full_bar[warp][s], parity)) failed = true;
    if (__any_sync(0xffffffffu, failed)) {
      failed = true;
      break;
    }
    const uint4* src = reinterpret_cast<const uint4*>(my_tiles_smem + s * kTileElems);
    uint4* dst = reinterpret_cast<uint4*>(out + t * kTileElems);
    for (uint32_t q = lane; q < quanta; q += 32) {
      A acc[kQ];
#pragma unroll
      for (int v = 0; v < kNI; ++v) VecIO<TI>::Load(src[q * kNI + v], acc + v * VecIO<TI>::kN);
      if (do_scale) {
#pragma unroll
        for (int e = 0; e < kQ; ++e) acc[e] = ScaleAcc<A>(acc[e], scale);
      }
      typename Acc<TO>::type out_acc[kQ];
#pragma unroll
      for (int e = 0; e < kQ; ++e) out_acc[e] = static_cast<typename Acc<TO>::type>(acc[e]);
#pragma unroll
      for (int v = 0; v < kNO; ++v) St16(dst + q * kNO + v, VecIO<TO>::Store(out_acc + v * VecIO<TO>::kN));
    }
    // Every lane is done reading the stage before it is refilled.
    __syncwarp();
    if (lane == 0) {
      const uint64_t kn = k + kCopyStages;
      if (kn < my_tiles) {
        const uint64_t tn = first + kn * step;
        const uint32_t bytes = tile_elems(tn) * static_cast<uint32_t>(sizeof(TI));
        MbarExpectTx(&full_bar[warp][s], bytes);
        BulkLoad(my_tiles_smem + s * kTileElems, in + tn * kTileElems, bytes, &full_bar[warp][s]);
      }
    }
  }
  if (failed && lane == 0 && doorbell != nullptr) *reinterpret_cast<volatile uint32_t*>(doorbell) = kStatusWaitTimeout;
  // Ragged end.
  if (blockIdx.x == 0) {
    for (uint64_t i = n_bulk + threadIdx.x; i < n; i += kCopyThreads) {
      A v = ToAcc<A, TI>(in[i]);
      out[i] = FromAcc<TO, A>(ScaleAcc<A>(v, scale));
    }
  }
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
  const size_t smem = static_cast<size_t>(dev::kCopyWarps) * dev::kCopyStages * dev::kCopyTileBytesIn;
  // The opt-in to more than 48 KiB of dynamic shared memory is a property of
  // the (function, device) pair and the call is cheap: made on every launch,
  // so a thread that moves to another GPU is covered.
  {
    cudaError_t e = cudaFuncSetAttribute(dev::CopyScaleTmaKernel<TI, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return e;
  }
  if (const char* e = getenv("IBCOMM_COPY_BLOCKS")) {  // experiment knob: CTAs of the copy kernel
    int v = atoi(e);
    if (v > 0) blocks = v;
  }
  const uint64_t tiles = (p.len_elements + kTileElems - 1) / kTileElems;
  const uint64_t blocks_needed = (tiles + dev::kCopyWarps - 1) / dev::kCopyWarps;
  if (static_cast<uint64_t>(blocks) > blocks_needed) blocks = static_cast<int>(blocks_needed);
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
