// Element access for the HBM-streaming row kernels: one element, or eight consecutive elements (16 bytes of bf16 /
// fp16, 32 bytes of fp32) of a row, as floats.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

#include <type_traits>

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

// eight packed elements (one 16-byte word of bf16 / fp16) to floats and back: two elements per 32-bit word, the
// conversions written out so that each pair costs two (bf16: a shift and a mask) resp. one instruction
template <typename T>
__device__ __forceinline__ void unpack8(const uint4& u, float (&x)[8]) {
  static_assert(sizeof(T) == 2, "16-bit element types");
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if constexpr (!std::is_same<T, __half>::value) {
      x[2 * i] = __uint_as_float(w[i] << 16);
      x[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    } else {
      const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
      x[2 * i] = f.x;
      x[2 * i + 1] = f.y;
    }
  }
}
template <typename T>
__device__ __forceinline__ uint4 pack8(const float (&x)[8]) {
  static_assert(sizeof(T) == 2, "16-bit element types");
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if constexpr (!std::is_same<T, __half>::value) {
      const __nv_bfloat162 p = __floats2bfloat162_rn(x[2 * i], x[2 * i + 1]);
      w[i] = *reinterpret_cast<const uint32_t*>(&p);
    } else {
      const __half2 p = __floats2half2_rn(x[2 * i], x[2 * i + 1]);
      w[i] = *reinterpret_cast<const uint32_t*>(&p);
    }
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}

// 8 consecutive elements of a row as floats (16 bytes of bf16 / fp16, 32 bytes of fp32)
template <typename T>
__device__ __forceinline__ void load8(const void* base, int64_t idx, float (&x)[8]) {
  if constexpr (sizeof(T) == 2) {
    unpack8<T>(*reinterpret_cast<const uint4*>(static_cast<const T*>(base) + idx), x);
  } else {
    const float4 a = *reinterpret_cast<const float4*>(static_cast<const float*>(base) + idx);
    const float4 b = *reinterpret_cast<const float4*>(static_cast<const float*>(base) + idx + 4);
    x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w; x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
  }
}
template <typename T>
__device__ __forceinline__ void store8(void* base, int64_t idx, const float (&x)[8]) {
  if constexpr (sizeof(T) == 2) {
    *reinterpret_cast<uint4*>(static_cast<T*>(base) + idx) = pack8<T>(x);
  } else {
    *reinterpret_cast<float4*>(static_cast<float*>(base) + idx) = make_float4(x[0], x[1], x[2], x[3]);
    *reinterpret_cast<float4*>(static_cast<float*>(base) + idx + 4) = make_float4(x[4], x[5], x[6], x[7]);
  }
}

// the same for C = 4 or 8 consecutive elements
template <typename T, int C>
__device__ __forceinline__ void load_c(const void* base, int64_t idx, float (&x)[C]) {
  static_assert(C == 4 || C == 8, "four or eight elements");
  if constexpr (C == 8) {
    load8<T>(base, idx, x);
  } else if constexpr (sizeof(T) == 2) {
    const uint2 u = *reinterpret_cast<const uint2*>(static_cast<const T*>(base) + idx);
    float y[8];
    unpack8<T>(make_uint4(u.x, u.y, 0u, 0u), y);
#pragma unroll
    for (int i = 0; i < 4; ++i) x[i] = y[i];
  } else {
    const float4 a = *reinterpret_cast<const float4*>(static_cast<const float*>(base) + idx);
    x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w;
  }
}
template <typename T, int C>
__device__ __forceinline__ void store_c(void* base, int64_t idx, const float (&x)[C]) {
  static_assert(C == 4 || C == 8, "four or eight elements");
  if constexpr (C == 8) {
    store8<T>(base, idx, x);
  } else if constexpr (sizeof(T) == 2) {
    const float y[8] = {x[0], x[1], x[2], x[3], 0.f, 0.f, 0.f, 0.f};
    const uint4 u = pack8<T>(y);
    *reinterpret_cast<uint2*>(static_cast<T*>(base) + idx) = make_uint2(u.x, u.y);
  } else {
    *reinterpret_cast<float4*>(static_cast<float*>(base) + idx) = make_float4(x[0], x[1], x[2], x[3]);
  }
}

// sigmoid with two MUFU instructions (ex2.approx.ftz, rcp.approx.ftz: about 2 ulp each; the library forms of exp and
// division add range handling that costs more instructions than the rest of an element's work in these kernels)
__device__ __forceinline__ float fast_sigmoid(float x) {
  float e, r;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(e) : "f"(x * -1.4426950408889634f));
  asm("rcp.approx.ftz.f32 %0, %1;\n" : "=f"(r) : "f"(1.f + e));
  return r;
}

}  // namespace gdn
