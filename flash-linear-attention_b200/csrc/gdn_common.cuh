// Shared device helpers and host-side launch plumbing for the gated-delta-rule kernels (sm_100a): chunk tables,
// bf16 packing, small asynchronous copies, the per-chunk gate vector, the L2 look-ahead, launch prototypes.
// (The tensor-core / TMEM / TMA primitives live in tc5.cuh, tc5_tile.cuh and tma.cuh.)
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/b200gdn.h"

namespace gdn {

constexpr int BT = 64;   // tokens per chunk

struct ChunkMeta {
  int seq, row, len, local;
};

__device__ __forceinline__ ChunkMeta load_chunk_meta(const int32_t* chunk_meta, int c) {
  int4 m = reinterpret_cast<const int4*>(chunk_meta)[c];
  return ChunkMeta{m.x, m.y, m.z, m.w};
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---- small asynchronous global -> shared copies (4 bytes per thread) --------------------------------------
__device__ __forceinline__ void cp_async4(void* smem, const void* gmem) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(smem_u32(smem)), "l"(gmem));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}

// ---- bf16 pairs ------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float2 unpack_bf16(uint32_t v) {
  __nv_bfloat162 b = *reinterpret_cast<__nv_bfloat162*>(&v);
  return __bfloat1622float2(b);
}

// Shared address of the 16-byte chunk holding (row r, columns col8 .. col8+7) of a bf16 tile of `rows` rows in the
// 128-byte-swizzled panel layout (what TMA writes and the tensor cores read).
__device__ __forceinline__ uint32_t swz_chunk_addr(uint32_t tile, int rows, int r, int col8) {
  return tile + (col8 >> 6) * (rows * 128) + r * 128 + ((((col8 >> 3) & 7) ^ (r & 7)) << 4);
}

// gamma is stored per chunk, [n_chunks][HV][64] fp32, entries past the chunk's valid length repeating the
// last valid value (so 2^(gamma_last - gamma_i) is 1 there): a chunk's 64 values are 256 contiguous,
// 256-byte aligned bytes that one bulk copy or one coalesced load brings in.
__device__ __forceinline__ const float* gamma_ptr(const float* gamma, int c, int HV, int hv) {
  return gamma + ((int64_t)c * HV + hv) * BT;
}

// Look-ahead for the one-CTA-per-(chunk, head) kernels.  CTAs are dispatched in launch order (x fastest), so the
// CTA that will take this one's place on the device is `dist` CTAs further on (dist = CTAs resident at once).
// A CTA pulls that successor's tiles into L2 as it starts; the successor's own loads then see L2 latency
// instead of DRAM latency.  Returns false when there is no successor.
__device__ __forceinline__ bool successor_cta(int dist, int& c2, int& h2) {
  const int nxt = blockIdx.y * gridDim.x + blockIdx.x + dist;
  if (nxt >= (int)(gridDim.x * gridDim.y)) return false;
  c2 = nxt % gridDim.x;
  h2 = nxt / gridDim.x;
  return true;
}

}  // namespace gdn

// ---- host-side launch plumbing (one translation unit per kernel, collected by api.cu) ---------------
namespace gdn {
int launch_intra_fwd(const b200gdn_chunk_args& a, cudaStream_t st);
int launch_scan_fwd(const b200gdn_chunk_args& a, cudaStream_t st);
int launch_scan_out_fwd(const b200gdn_chunk_args& a, cudaStream_t st);
int launch_out_fwd(const b200gdn_chunk_args& a, cudaStream_t st);
int launch_dv_local(const b200gdn_chunk_args& a, cudaStream_t st);
int launch_scan_bwd(const b200gdn_chunk_args& a, cudaStream_t st);
int launch_scan_dvl_bwd(const b200gdn_chunk_args& a, cudaStream_t st);
int launch_bwd_dqk(const b200gdn_chunk_args& a, cudaStream_t st);
int launch_bwd_wy(const b200gdn_chunk_args& a, cudaStream_t st);
int launch_recurrent(const b200gdn_recurrent_args& a, cudaStream_t st);
int launch_affine(const b200gdn_affine_args& a, cudaStream_t st);
int launch_cp_fold(const b200gdn_fold_args& a, cudaStream_t st);
int launch_cp_prefix(const b200gdn_prefix_args& a, cudaStream_t st);
int launch_prep(const b200gdn_prep_args& a, cudaStream_t st, bool bwd);
int launch_conv(const b200gdn_conv_args& a, cudaStream_t st, bool bwd);
int launch_norm_gate(const b200gdn_norm_gate_args& a, cudaStream_t st, bool bwd);
int norm_gate_grid(int64_t rows);
int decode_timeout_flag();
int intra_fwd_timeout_flag();
int scan_fwd_timeout_flag();
int out_fwd_timeout_flag();
int dv_local_timeout_flag();
int scan_bwd_timeout_flag();
int bwd_dqk_timeout_flag();
int bwd_wy_timeout_flag();
int set_error(int code, const char* fmt, ...);
int check_launch(const char* what);
void reset_launch_count();

template <typename Kern>
int ensure_smem(Kern kern, size_t bytes) {
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
  if (e != cudaSuccess) return set_error(B200GDN_ERR_CUDA, "cudaFuncSetAttribute(%zu B): %s", bytes, cudaGetErrorString(e));
  return 0;
}

// CTAs of `kern` resident on the whole device at once (SMs x CTAs per SM); cached per instantiation and device.
template <typename Kern>
int resident_ctas(Kern kern, int threads, size_t smem) {
  static int cached[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && cached[dev] > 0) return cached[dev];
  int per_sm = 1, sms = 148;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, threads, smem) != cudaSuccess || per_sm < 1) per_sm = 1;
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms < 1) sms = 148;
  if (dev >= 0 && dev < 64) cached[dev] = per_sm * sms;
  return per_sm * sms;
}
}  // namespace gdn
