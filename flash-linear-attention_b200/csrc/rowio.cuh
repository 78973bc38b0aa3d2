// Element access for the HBM-streaming row kernels: one element, or eight consecutive elements (16 bytes of bf16 /
// fp16, 32 bytes of fp32) of a row, as floats.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

namespace gdn {

template <typename T> struct Io;
template <> struct Io<__nv_bfloat16> {
  static __device__ __forceinline__ float ld(const void* p, int64_t i) { return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]); }
  static __device__ __forceinline__ void st(void* p, int64_t i, float v) { static_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v); }
};
template <> struct Io<__half> {
  static __device__ __forceinline__ float ld(const void* p, int64_t i) { return __half2float(static_cast<const __half*>(p)[i]); }
  static __device__ __forceinline__ void st(void* p, int64_t i, float v) { static_cast<__half*>(p)[i] = __float2half_rn(v); }
};
template <> struct Io<float> {
  static __device__ __forceinline__ float ld(const void* p, int64_t i) { return static_cast<const float*>(p)[i]; }
  static __device__ __forceinline__ void st(void* p, int64_t i, float v) { static_cast<float*>(p)[i] = v; }
};

// 8 consecutive elements of a row as floats (16 bytes of bf16 / fp16, 32 bytes of fp32)
template <typename T>
__device__ __forceinline__ void load8(const void* base, int64_t idx, float (&x)[8]) {
  if constexpr (sizeof(T) == 2) {
    const uint4 u = *reinterpret_cast<const uint4*>(static_cast<const T*>(base) + idx);
    const T* e = reinterpret_cast<const T*>(&u);
#pragma unroll
    for (int i = 0; i < 8; ++i) x[i] = Io<T>::ld(e, i);
  } else {
    const float4 a = *reinterpret_cast<const float4*>(static_cast<const float*>(base) + idx);
    const float4 b = *reinterpret_cast<const float4*>(static_cast<const float*>(base) + idx + 4);
    x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w; x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
  }
}
template <typename T>
__device__ __forceinline__ void store8(void* base, int64_t idx, const float (&x)[8]) {
  if constexpr (sizeof(T) == 2) {
    uint4 u;
    T* e = reinterpret_cast<T*>(&u);
#pragma unroll
    for (int i = 0; i < 8; ++i) Io<T>::st(e, i, x[i]);
    *reinterpret_cast<uint4*>(static_cast<T*>(base) + idx) = u;
  } else {
    *reinterpret_cast<float4*>(static_cast<float*>(base) + idx) = make_float4(x[0], x[1], x[2], x[3]);
    *reinterpret_cast<float4*>(static_cast<float*>(base) + idx + 4) = make_float4(x[4], x[5], x[6], x[7]);
  }
}

}  // namespace gdn
