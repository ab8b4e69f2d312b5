// Device-buffer allreduce templates.  Same signatures as the reference
// (ibcomm/allreduce_cuda_impl.h:35-36, 326-327); the element type selects a
// kernel instantiation instead of a generic grid-stride `+=` loop.  Calls
// return when the result is in recvbuf, like the reference's.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <type_traits>

#include "ibcomm/communicator.h"

namespace ibcomm {

template <typename T> struct DTypeOf;
template <> struct DTypeOf<float> { static constexpr DType value = DType::kFloat32; };
template <> struct DTypeOf<double> { static constexpr DType value = DType::kFloat64; };
template <> struct DTypeOf<int> { static constexpr DType value = DType::kInt32; };
template <> struct DTypeOf<unsigned int> { static constexpr DType value = DType::kInt32; };
template <> struct DTypeOf<long long> { static constexpr DType value = DType::kInt64; };
template <> struct DTypeOf<long> { static constexpr DType value = sizeof(long) == 8 ? DType::kInt64 : DType::kInt32; };
template <> struct DTypeOf<__half> { static constexpr DType value = DType::kFloat16; };
template <> struct DTypeOf<__nv_bfloat16> { static constexpr DType value = DType::kBFloat16; };

template <typename T>
void Communicator::AllreduceRingCuda(const T* sendbuf, T* recvbuf, size_t len_elements) {
  CudaAllreduceOptions o;
  o.algo = Algo::kRing;
  AllreduceCuda(DTypeOf<T>::value, sendbuf, recvbuf, len_elements, o);
}

template <typename T>
void Communicator::ReduceScatterCuda(const T* sendbuf, T* recvbuf, size_t block_elements) {
  ReduceScatterCuda(DTypeOf<T>::value, sendbuf, recvbuf, block_elements, CudaAllreduceOptions());
}

template <typename T>
void Communicator::AllGatherCuda(const T* sendbuf, T* recvbuf, size_t block_elements) {
  AllGatherCuda(DTypeOf<T>::value, sendbuf, recvbuf, block_elements, CudaAllreduceOptions());
}

template <typename T>
void Communicator::AllreduceRabenseifnerCuda(const T* sendbuf, T* recvbuf, size_t len_elements) {
  CudaAllreduceOptions o;
  o.algo = Algo::kRabenseifner;
  AllreduceCuda(DTypeOf<T>::value, sendbuf, recvbuf, len_elements, o);
}

}  // namespace ibcomm
