// TMA (cp.async.bulk.tensor) helpers: host-side tensor-map encoding without linking libcuda, and the
// device-side load / store / group instructions.  Every tile moved here is a box of 64 bf16 columns
// (128 bytes) by up to 256 rows with the 128-byte swizzle, i.e. exactly one "panel" of the shared
// layout described in tc5.cuh.  No cluster-wide copies are used anywhere: every copy targets the
// issuing CTA's own shared memory.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace tma {

// ---- host ----------------------------------------------------------------------------------------------
// 2-D map over a row-major bf16 matrix [rows][cols] (row pitch `pitch_elems` elements), box = 64 columns x
// `box_rows` rows, 128-byte swizzle, zero fill outside the matrix.
// Returns 0 on success, otherwise the CUresult / a negative value when the driver entry point is missing.
inline int encode_bf16_2d(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint64_t pitch_elems,
                          uint32_t box_rows) {
  typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                               const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                               CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  static EncodeFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || p == nullptr) return -1;
    fn = reinterpret_cast<EncodeFn>(p);
  }
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {pitch_elems * 2};
  cuuint32_t box[2] = {64, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return static_cast<int>(r);
}

// 3-D "panel" view of the same kind of matrix: dimension 0 = 64 columns of one panel, dimension 1 = rows,
// dimension 2 = panel index (cols / 64, 128 bytes apart).  A box {64, box_rows, box_panels} lands in
// shared memory panel after panel, i.e. a [box_rows][64 * box_panels] tile in the panel layout of
// tc5.cuh arrives with ONE copy instruction.
inline int encode_bf16_panels(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint64_t pitch_elems,
                              uint32_t box_rows, uint32_t box_panels) {
  typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                               const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                               CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  static EncodeFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || p == nullptr) return -1;
    fn = reinterpret_cast<EncodeFn>(p);
  }
  cuuint64_t dims[3] = {64, rows, cols / 64};
  cuuint64_t strides[2] = {pitch_elems * 2, 128};
  cuuint32_t box[3] = {64, box_rows, box_panels};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return static_cast<int>(r);
}

// ---- device --------------------------------------------------------------------------------------------
#ifdef __CUDACC__
__device__ __forceinline__ uint32_t saddr(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

// global -> shared box at column x (elements, multiple of 8), row y; completion is signalled on `bar` (bytes).
__device__ __forceinline__ void load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n" ::"r"(
          saddr(dst)),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(saddr(bar)), "r"(x), "r"(y)
      : "memory");
}
// panel view: row y, first panel z
__device__ __forceinline__ void load_3d(void* dst, const CUtensorMap* map, int y, int z, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];\n" ::"r"(
          saddr(dst)),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(saddr(bar)), "r"(0), "r"(y), "r"(z)
      : "memory");
}
__device__ __forceinline__ void store_3d(const CUtensorMap* map, int y, int z, const void* src) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];\n" ::"l"(
                   reinterpret_cast<uint64_t>(map)),
               "r"(saddr(src)), "r"(0), "r"(y), "r"(z)
               : "memory");
}
// plain contiguous copy global -> shared (both 16-byte aligned, size a multiple of 16)
__device__ __forceinline__ void load_1d(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(saddr(dst)),
               "l"(src), "r"(bytes), "r"(saddr(bar))
               : "memory");
}
// shared -> global box; joins the current bulk group of the issuing thread.
__device__ __forceinline__ void store_2d(const CUtensorMap* map, int x, int y, const void* src) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];\n" ::"l"(
                   reinterpret_cast<uint64_t>(map)),
               "r"(saddr(src)), "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void store_commit() { asm volatile("cp.async.bulk.commit_group;\n" ::: "memory"); }
// wait until at most N of this thread's bulk groups still READ their shared source
template <int N>
__device__ __forceinline__ void store_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;\n" ::"n"(N) : "memory");
}
template <int N>
__device__ __forceinline__ void store_wait_all() {
  asm volatile("cp.async.bulk.wait_group %0;\n" ::"n"(N) : "memory");
}
// pull a box into L2 only (no shared-memory destination, no completion): a later load of the same box is short
__device__ __forceinline__ void prefetch_2d(const CUtensorMap* map, int x, int y) {
  asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global [%0, {%1, %2}];\n" ::"l"(reinterpret_cast<uint64_t>(map)), "r"(x),
               "r"(y)
               : "memory");
}
// the same for a box of the panel view (row y, first panel z)
__device__ __forceinline__ void prefetch_3d(const CUtensorMap* map, int y, int z) {
  asm volatile("cp.async.bulk.prefetch.tensor.3d.L2.global [%0, {%1, %2, %3}];\n" ::"l"(reinterpret_cast<uint64_t>(map)),
               "r"(0), "r"(y), "r"(z)
               : "memory");
}
// one 128-byte line of plain global memory into L2
__device__ __forceinline__ void prefetch_line(const void* p) { asm volatile("prefetch.global.L2 [%0];\n" ::"l"(p)); }
__device__ __forceinline__ void prefetch_map(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];\n" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}
#endif

}  // namespace tma
