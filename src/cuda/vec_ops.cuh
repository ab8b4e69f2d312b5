// Element-type traits and 16-byte vector accesses for the reduction kernels.
// Sums of 16-bit floats are accumulated in fp32; fp32 buffers may travel as
// bf16 or fp16 on the wire.  Everything here works on uint4 values held in
// registers: VecIO<X> unpacks one 16-byte vector of X into accumulators, adds
// one to accumulators, or packs accumulators back.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cstdint>

namespace ibcomm {
namespace dev {

template <typename T> struct Acc { using type = T; };
template <> struct Acc<__half> { using type = float; };
template <> struct Acc<__nv_bfloat16> { using type = float; };

template <typename A, typename T> __device__ __forceinline__ A ToAcc(T v) { return static_cast<A>(v); }
template <> __device__ __forceinline__ float ToAcc<float, __half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float ToAcc<float, __nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T, typename A> __device__ __forceinline__ T FromAcc(A v) { return static_cast<T>(v); }
template <> __device__ __forceinline__ __half FromAcc<__half, float>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 FromAcc<__nv_bfloat16, float>(float v) { return __float2bfloat16_rn(v); }

template <typename A> __device__ __forceinline__ A ScaleAcc(A v, double s) { return static_cast<A>(v * static_cast<A>(s)); }
template <> __device__ __forceinline__ float ScaleAcc<float>(float v, double s) { return v * static_cast<float>(s); }
template <> __device__ __forceinline__ int ScaleAcc<int>(int v, double s) { return static_cast<int>(static_cast<double>(v) * s); }
template <> __device__ __forceinline__ long long ScaleAcc<long long>(long long v, double s) {
  return static_cast<long long>(static_cast<double>(v) * s);
}

// Raw 16-byte accesses.  "Strong" loads bypass L1 (data written by a peer
// over NVLink); weak loads may be cached.
__device__ __forceinline__ uint4 Ld16Strong(const void* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint4 Ld16(const void* p) {
  uint4 v;
  asm volatile("ld.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void St16(void* p, uint4 v) {
  asm volatile("st.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

template <typename X> struct VecIO;

template <> struct VecIO<float> {
  static constexpr int kN = 4;
  __device__ __forceinline__ static void Load(uint4 q, float* a) {
    a[0] = __uint_as_float(q.x); a[1] = __uint_as_float(q.y); a[2] = __uint_as_float(q.z); a[3] = __uint_as_float(q.w);
  }
  __device__ __forceinline__ static void Add(uint4 q, float* a) {
    a[0] += __uint_as_float(q.x); a[1] += __uint_as_float(q.y); a[2] += __uint_as_float(q.z); a[3] += __uint_as_float(q.w);
  }
  __device__ __forceinline__ static uint4 Store(const float* a) {
    return make_uint4(__float_as_uint(a[0]), __float_as_uint(a[1]), __float_as_uint(a[2]), __float_as_uint(a[3]));
  }
};

template <> struct VecIO<int> {
  static constexpr int kN = 4;
  __device__ __forceinline__ static void Load(uint4 q, int* a) {
    a[0] = static_cast<int>(q.x); a[1] = static_cast<int>(q.y); a[2] = static_cast<int>(q.z); a[3] = static_cast<int>(q.w);
  }
  __device__ __forceinline__ static void Add(uint4 q, int* a) {
    a[0] += static_cast<int>(q.x); a[1] += static_cast<int>(q.y); a[2] += static_cast<int>(q.z); a[3] += static_cast<int>(q.w);
  }
  __device__ __forceinline__ static uint4 Store(const int* a) {
    return make_uint4(static_cast<unsigned>(a[0]), static_cast<unsigned>(a[1]), static_cast<unsigned>(a[2]), static_cast<unsigned>(a[3]));
  }
};

template <> struct VecIO<double> {
  static constexpr int kN = 2;
  __device__ __forceinline__ static double D(unsigned lo, unsigned hi) { return __hiloint2double(static_cast<int>(hi), static_cast<int>(lo)); }
  __device__ __forceinline__ static void Load(uint4 q, double* a) { a[0] = D(q.x, q.y); a[1] = D(q.z, q.w); }
  __device__ __forceinline__ static void Add(uint4 q, double* a) { a[0] += D(q.x, q.y); a[1] += D(q.z, q.w); }
  __device__ __forceinline__ static uint4 Store(const double* a) {
    return make_uint4(static_cast<unsigned>(__double2loint(a[0])), static_cast<unsigned>(__double2hiint(a[0])),
                      static_cast<unsigned>(__double2loint(a[1])), static_cast<unsigned>(__double2hiint(a[1])));
  }
};

template <> struct VecIO<long long> {
  static constexpr int kN = 2;
  __device__ __forceinline__ static long long L(unsigned lo, unsigned hi) {
    return static_cast<long long>((static_cast<unsigned long long>(hi) << 32) | lo);
  }
  __device__ __forceinline__ static void Load(uint4 q, long long* a) { a[0] = L(q.x, q.y); a[1] = L(q.z, q.w); }
  __device__ __forceinline__ static void Add(uint4 q, long long* a) { a[0] += L(q.x, q.y); a[1] += L(q.z, q.w); }
  __device__ __forceinline__ static uint4 Store(const long long* a) {
    unsigned long long u0 = static_cast<unsigned long long>(a[0]), u1 = static_cast<unsigned long long>(a[1]);
    return make_uint4(static_cast<unsigned>(u0), static_cast<unsigned>(u0 >> 32), static_cast<unsigned>(u1), static_cast<unsigned>(u1 >> 32));
  }
};

template <> struct VecIO<__half> {
  static constexpr int kN = 8;
  __device__ __forceinline__ static float2 H2(unsigned w) {
    __half2 h = *reinterpret_cast<__half2*>(&w);
    return __half22float2(h);
  }
  __device__ __forceinline__ static unsigned P2(float a, float b) {
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<unsigned*>(&h);
  }
  __device__ __forceinline__ static void Load(uint4 q, float* a) {
    float2 f;
    f = H2(q.x); a[0] = f.x; a[1] = f.y;
    f = H2(q.y); a[2] = f.x; a[3] = f.y;
    f = H2(q.z); a[4] = f.x; a[5] = f.y;
    f = H2(q.w); a[6] = f.x; a[7] = f.y;
  }
  __device__ __forceinline__ static void Add(uint4 q, float* a) {
    float2 f;
    f = H2(q.x); a[0] += f.x; a[1] += f.y;
    f = H2(q.y); a[2] += f.x; a[3] += f.y;
    f = H2(q.z); a[4] += f.x; a[5] += f.y;
    f = H2(q.w); a[6] += f.x; a[7] += f.y;
  }
  __device__ __forceinline__ static uint4 Store(const float* a) {
    return make_uint4(P2(a[0], a[1]), P2(a[2], a[3]), P2(a[4], a[5]), P2(a[6], a[7]));
  }
};

template <> struct VecIO<__nv_bfloat16> {
  static constexpr int kN = 8;
  // bf16 is the upper half of an fp32 bit pattern.
  __device__ __forceinline__ static float Lo(unsigned w) { return __uint_as_float(w << 16); }
  __device__ __forceinline__ static float Hi(unsigned w) { return __uint_as_float(w & 0xffff0000u); }
  __device__ __forceinline__ static unsigned P2(float a, float b) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<unsigned*>(&h);
  }
  __device__ __forceinline__ static void Load(uint4 q, float* a) {
    a[0] = Lo(q.x); a[1] = Hi(q.x); a[2] = Lo(q.y); a[3] = Hi(q.y);
    a[4] = Lo(q.z); a[5] = Hi(q.z); a[6] = Lo(q.w); a[7] = Hi(q.w);
  }
  __device__ __forceinline__ static void Add(uint4 q, float* a) {
    a[0] += Lo(q.x); a[1] += Hi(q.x); a[2] += Lo(q.y); a[3] += Hi(q.y);
    a[4] += Lo(q.z); a[5] += Hi(q.z); a[6] += Lo(q.w); a[7] += Hi(q.w);
  }
  __device__ __forceinline__ static uint4 Store(const float* a) {
    return make_uint4(P2(a[0], a[1]), P2(a[2], a[3]), P2(a[4], a[5]), P2(a[6], a[7]));
  }
};

template <typename X> __device__ __forceinline__ X LdScalarStrong(const X* p) {
  return *reinterpret_cast<const volatile X*>(p);
}
template <> __device__ __forceinline__ __half LdScalarStrong<__half>(const __half* p) {
  unsigned short u = *reinterpret_cast<const volatile unsigned short*>(p);
  return __ushort_as_half(u);
}
template <> __device__ __forceinline__ __nv_bfloat16 LdScalarStrong<__nv_bfloat16>(const __nv_bfloat16* p) {
  unsigned short u = *reinterpret_cast<const volatile unsigned short*>(p);
  return __ushort_as_bfloat16(u);
}

}  // namespace dev
}  // namespace ibcomm
