// Shared device helpers for the gated-delta-rule kernels (sm_100a).
//
// Tiles are 64 tokens (one chunk) by a head dimension, staged in shared memory as bf16 with a row
// stride of (cols + 8) elements so that the eight 16-byte rows an ldmatrix touches fall in distinct
// banks.  Warp-level contractions use mma.sync m16n8k16 (bf16 in, fp32 accumulate); operand
// fragments are fetched with ldmatrix, transposed by the instruction where the contraction needs
// the other major-ness, never by a physical transpose.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/b200gdn.h"

namespace gdn {

constexpr int BT = 64;
constexpr int PAD = 8;  // bf16 elements of row padding

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

// ---- async global -> shared copies (16 bytes; zero-fill when !pred) -------------------------------
__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool pred) {
  uint32_t s = smem_u32(smem);
  int bytes = pred ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void cp_async4(void* smem, const void* gmem) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(smem_u32(smem)), "l"(gmem));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}

// Copy a [64][COLS] bf16 tile (global row stride `gstride` elements) into shared memory with row
// stride COLS+PAD; rows >= valid are zero-filled.  `src` points at (first row, first column).
template <int COLS, int NTHREADS>
__device__ __forceinline__ void load_tile_async(__nv_bfloat16* dst, const __nv_bfloat16* src, int64_t gstride,
                                                int valid, int tid) {
  constexpr int CPR = COLS / 8;  // 16-byte chunks per row
  constexpr int TOTAL = BT * CPR;
  static_assert(TOTAL % NTHREADS == 0, "tile/threads mismatch");
#pragma unroll
  for (int it = 0; it < TOTAL / NTHREADS; ++it) {
    int idx = it * NTHREADS + tid;
    int r = idx / CPR, c = idx % CPR;
    bool ok = r < valid;
    const __nv_bfloat16* g = src + (ok ? (int64_t)r * gstride : 0) + c * 8;
    cp_async16(dst + r * (COLS + PAD) + c * 8, g, ok);
  }
}

// Same for a [ROWS][COLS] tile that is always fully valid (state snapshots).
template <int ROWS, int COLS, int NTHREADS>
__device__ __forceinline__ void load_rows_async(__nv_bfloat16* dst, const __nv_bfloat16* src, int64_t gstride,
                                                int tid) {
  constexpr int CPR = COLS / 8;
  constexpr int TOTAL = ROWS * CPR;
  static_assert(TOTAL % NTHREADS == 0, "tile/threads mismatch");
#pragma unroll
  for (int it = 0; it < TOTAL / NTHREADS; ++it) {
    int idx = it * NTHREADS + tid;
    int r = idx / CPR, c = idx % CPR;
    cp_async16(dst + r * (COLS + PAD) + c * 8, src + (int64_t)r * gstride + c * 8, true);
  }
}

// Write a [ROWS][COLS] bf16 tile from shared memory (row stride COLS+PAD) to global, 16 bytes per
// thread and access, rows < valid only.
template <int ROWS, int COLS, int NTHREADS>
__device__ __forceinline__ void store_tile(__nv_bfloat16* dst, int64_t gstride, const __nv_bfloat16* src, int valid,
                                           int tid) {
  constexpr int CPR = COLS / 8;
  constexpr int TOTAL = ROWS * CPR;
  static_assert(TOTAL % NTHREADS == 0, "tile/threads mismatch");
#pragma unroll
  for (int it = 0; it < TOTAL / NTHREADS; ++it) {
    int idx = it * NTHREADS + tid;
    int r = idx / CPR, c = idx % CPR;
    if (r < valid) {
      uint4 val = *reinterpret_cast<const uint4*>(src + r * (COLS + PAD) + c * 8);
      *reinterpret_cast<uint4*>(dst + (int64_t)r * gstride + c * 8) = val;
    }
  }
}

// ---- fragments -------------------------------------------------------------------------------------
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}

// A fragment (16 rows x 16 k) of a row-major operand As[m][k]; `p` points at (m0, k0).
__device__ __forceinline__ void load_a(uint32_t (&a)[4], const __nv_bfloat16* p, int ld, int lane) {
  ldsm_x4(a, smem_u32(p + (lane & 15) * ld + ((lane >> 4) << 3)));
}
// A fragment of an operand stored transposed, As[k][m]; `p` points at (k0, m0).
__device__ __forceinline__ void load_a_t(uint32_t (&a)[4], const __nv_bfloat16* p, int ld, int lane) {
  ldsm_x4_t(a, smem_u32(p + ((lane & 7) + ((lane >> 4) << 3)) * ld + (((lane >> 3) & 1) << 3)));
}
// B fragments for two adjacent n-tiles (16 k x 16 n) of an operand stored Bs[n][k]; `p` at (n0, k0).
// b[0],b[1] feed n-tile 0 and b[2],b[3] n-tile 1.
__device__ __forceinline__ void load_b_nk(uint32_t (&b)[4], const __nv_bfloat16* p, int ld, int lane) {
  ldsm_x4(b, smem_u32(p + ((lane & 7) + ((lane >> 4) << 3)) * ld + (((lane >> 3) & 1) << 3)));
}
// B fragments for two adjacent n-tiles of an operand stored Bs[k][n]; `p` at (k0, n0).
__device__ __forceinline__ void load_b_kn(uint32_t (&b)[4], const __nv_bfloat16* p, int ld, int lane) {
  ldsm_x4_t(b, smem_u32(p + ((lane & 7) + (((lane >> 3) & 1) << 3)) * ld + ((lane >> 4) << 3)));
}

__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float2 unpack_bf16(uint32_t v) {
  __nv_bfloat162 b = *reinterpret_cast<__nv_bfloat162*>(&v);
  return __bfloat1622float2(b);
}

// ---- the same fragments from tiles in the 128-byte-swizzled panel layout (what TMA writes) -----------
// A tile of `rows` rows is a stack of 64-column panels (rows*128 bytes each); inside a panel row r
// starts at r*128 and its 16-byte chunk c sits at position c ^ (r & 7).  Every ldmatrix lane fetches one
// chunk, so the swizzle is applied per lane and the eight rows of a matrix hit distinct banks.
__device__ __forceinline__ uint32_t swz_chunk_addr(uint32_t tile, int rows, int r, int col8) {
  return tile + (col8 >> 6) * (rows * 128) + r * 128 + ((((col8 >> 3) & 7) ^ (r & 7)) << 4);
}
// `tile` is the shared-memory address (u32) of the tile; (m0, k0) etc. are element coordinates.
__device__ __forceinline__ void load_a_swz(uint32_t (&a)[4], uint32_t tile, int rows, int m0, int k0, int lane) {
  ldsm_x4(a, swz_chunk_addr(tile, rows, m0 + (lane & 15), k0 + ((lane >> 4) << 3)));
}
__device__ __forceinline__ void load_a_t_swz(uint32_t (&a)[4], uint32_t tile, int rows, int k0, int m0, int lane) {
  ldsm_x4_t(a, swz_chunk_addr(tile, rows, k0 + (lane & 7) + ((lane >> 4) << 3), m0 + (((lane >> 3) & 1) << 3)));
}
__device__ __forceinline__ void load_b_nk_swz(uint32_t (&b)[4], uint32_t tile, int rows, int n0, int k0, int lane) {
  ldsm_x4(b, swz_chunk_addr(tile, rows, n0 + (lane & 7) + ((lane >> 4) << 3), k0 + (((lane >> 3) & 1) << 3)));
}
__device__ __forceinline__ void load_b_kn_swz(uint32_t (&b)[4], uint32_t tile, int rows, int k0, int n0, int lane) {
  ldsm_x4_t(b, swz_chunk_addr(tile, rows, k0 + (lane & 7) + (((lane >> 3) & 1) << 3), n0 + ((lane >> 4) << 3)));
}
// 4-byte access to element pair (r, col), col even
__device__ __forceinline__ uint32_t swz_pair_addr(uint32_t tile, int rows, int r, int col) {
  return swz_chunk_addr(tile, rows, r, col & ~7) + ((col & 7) << 1);
}
__device__ __forceinline__ void sts32(uint32_t addr, uint32_t v) { asm volatile("st.shared.b32 [%0], %1;\n" ::"r"(addr), "r"(v)); }
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.b32 %0, [%1];\n" : "=r"(v) : "r"(addr));
  return v;
}

enum class AMajor { Row, Trans };
enum class BMajor { NK, KN };

// acc[NT][4] += A(16 x 16*KS) * B(16*KS x 8*NT) for one warp.
//  AMajor::Row   : As[m][k], pa -> (m0, 0)        AMajor::Trans : As[k][m], pa -> (0, m0)
//  BMajor::NK    : Bs[n][k], pb -> (n0, 0)        BMajor::KN    : Bs[k][n], pb -> (0, n0)
// NEG_A flips the sign of A (both bf16 halves) so that the product is subtracted.
// The operand fetches are software-pipelined by hand: the ldmatrix of step i+1 is issued before the
// MMAs of step i (the asm statements are volatile, so the compiler keeps this order), which takes the
// shared-memory latency off the dependent chain of MMAs.
template <int NT, int KS, AMajor AM, BMajor BM, bool NEG_A = false>
__device__ __forceinline__ void warp_mma(float (&acc)[NT][4], const __nv_bfloat16* pa, int lda, const __nv_bfloat16* pb,
                                         int ldb, int lane) {
  static_assert(NT % 2 == 0, "n-tiles come in pairs");
  constexpr int NP = NT / 2, STEPS = KS * NP;
  uint32_t a[2][4], b[2][4];
  auto ld_a = [&](int ks, uint32_t (&dst)[4]) {
    if (AM == AMajor::Row)
      load_a(dst, pa + ks * 16, lda, lane);
    else
      load_a_t(dst, pa + ks * 16 * lda, lda, lane);
    if (NEG_A) {
#pragma unroll
      for (int i = 0; i < 4; ++i) dst[i] ^= 0x80008000u;
    }
  };
  auto ld_b = [&](int ks, int np, uint32_t (&dst)[4]) {
    if (BM == BMajor::NK)
      load_b_nk(dst, pb + np * 16 * ldb + ks * 16, ldb, lane);
    else
      load_b_kn(dst, pb + ks * 16 * ldb + np * 16, ldb, lane);
  };
  ld_a(0, a[0]);
  ld_b(0, 0, b[0]);
#pragma unroll
  for (int st = 0; st < STEPS; ++st) {
    const int ks = st / NP, np = st % NP;
    if (st + 1 < STEPS) {
      const int ks1 = (st + 1) / NP, np1 = (st + 1) % NP;
      if (np1 == 0) ld_a(ks1, a[ks1 & 1]);
      ld_b(ks1, np1, b[(st + 1) & 1]);
    }
    mma16816(acc[2 * np], a[ks & 1], b[st & 1][0], b[st & 1][1]);
    mma16816(acc[2 * np + 1], a[ks & 1], b[st & 1][2], b[st & 1][3]);
  }
}

// The same contraction on swizzled tiles.  (am0, ak0) / (bn0, bk0) are the element coordinates of the
// operand blocks inside their tiles; the contraction runs over KS steps of 16 from ak0 / bk0.
template <int NT, int KS, AMajor AM, BMajor BM, bool NEG_A = false>
__device__ __forceinline__ void warp_mma_swz(float (&acc)[NT][4], uint32_t atile, int arows, int am0, int ak0, uint32_t btile,
                                             int brows, int bn0, int bk0, int lane) {
  static_assert(NT % 2 == 0, "n-tiles come in pairs");
  constexpr int NP = NT / 2, STEPS = KS * NP;
  uint32_t a[2][4], b[2][4];
  auto ld_a = [&](int ks, uint32_t (&dst)[4]) {
    if (AM == AMajor::Row)
      load_a_swz(dst, atile, arows, am0, ak0 + ks * 16, lane);
    else
      load_a_t_swz(dst, atile, arows, ak0 + ks * 16, am0, lane);
    if (NEG_A) {
#pragma unroll
      for (int i = 0; i < 4; ++i) dst[i] ^= 0x80008000u;
    }
  };
  auto ld_b = [&](int ks, int np, uint32_t (&dst)[4]) {
    if (BM == BMajor::NK)
      load_b_nk_swz(dst, btile, brows, bn0 + np * 16, bk0 + ks * 16, lane);
    else
      load_b_kn_swz(dst, btile, brows, bk0 + ks * 16, bn0 + np * 16, lane);
  };
  ld_a(0, a[0]);
  ld_b(0, 0, b[0]);
#pragma unroll
  for (int st = 0; st < STEPS; ++st) {
    const int ks = st / NP, np = st % NP;
    if (st + 1 < STEPS) {
      const int ks1 = (st + 1) / NP, np1 = (st + 1) % NP;
      if (np1 == 0) ld_a(ks1, a[ks1 & 1]);
      ld_b(ks1, np1, b[(st + 1) & 1]);
    }
    mma16816(acc[2 * np], a[ks & 1], b[st & 1][0], b[st & 1][1]);
    mma16816(acc[2 * np + 1], a[ks & 1], b[st & 1][2], b[st & 1][3]);
  }
}

// Store a warp's 16 x (8*NT) accumulator as bf16 into a swizzled tile at element (m0, n0).
template <int NT>
__device__ __forceinline__ void acc_to_swz(uint32_t tile, int rows, int m0, int n0, const float (&acc)[NT][4], int lane) {
  int g = lane >> 2, t = lane & 3;
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    sts32(swz_pair_addr(tile, rows, m0 + g, n0 + nt * 8 + 2 * t), pack_bf16(acc[nt][0], acc[nt][1]));
    sts32(swz_pair_addr(tile, rows, m0 + g + 8, n0 + nt * 8 + 2 * t), pack_bf16(acc[nt][2], acc[nt][3]));
  }
}

// Same with the A operand already in registers as KS fragments (a 16 x 16*KS bf16 matrix that was
// produced by a previous accumulator: see acc_to_afrag).
template <int NT, int KS, BMajor BM>
__device__ __forceinline__ void warp_mma_ra(float (&acc)[NT][4], const uint32_t (&afrag)[KS][4],
                                            const __nv_bfloat16* pb, int ldb, int lane) {
  constexpr int NP = NT / 2, STEPS = KS * NP;
  uint32_t b[2][4];
  auto ld_b = [&](int ks, int np, uint32_t (&dst)[4]) {
    if (BM == BMajor::NK)
      load_b_nk(dst, pb + np * 16 * ldb + ks * 16, ldb, lane);
    else
      load_b_kn(dst, pb + ks * 16 * ldb + np * 16, ldb, lane);
  };
  ld_b(0, 0, b[0]);
#pragma unroll
  for (int st = 0; st < STEPS; ++st) {
    const int ks = st / NP, np = st % NP;
    if (st + 1 < STEPS) ld_b((st + 1) / NP, (st + 1) % NP, b[(st + 1) & 1]);
    mma16816(acc[2 * np], afrag[ks], b[st & 1][0], b[st & 1][1]);
    mma16816(acc[2 * np + 1], afrag[ks], b[st & 1][2], b[st & 1][3]);
  }
}

// A 16 x (8*NT) fp32 accumulator, rounded to bf16, is exactly the A operand (16 x 16*(NT/2)) of the
// next contraction: thread (g = lane/4, t = lane%4) holds rows g, g+8 and columns 2t, 2t+1 of every
// n-tile, which is the m16n8k16 A layout when two n-tiles are paired.
template <int NT>
__device__ __forceinline__ void acc_to_afrag(uint32_t (&afrag)[NT / 2][4], const float (&acc)[NT][4]) {
#pragma unroll
  for (int ks = 0; ks < NT / 2; ++ks) {
    afrag[ks][0] = pack_bf16(acc[2 * ks][0], acc[2 * ks][1]);
    afrag[ks][1] = pack_bf16(acc[2 * ks][2], acc[2 * ks][3]);
    afrag[ks][2] = pack_bf16(acc[2 * ks + 1][0], acc[2 * ks + 1][1]);
    afrag[ks][3] = pack_bf16(acc[2 * ks + 1][2], acc[2 * ks + 1][3]);
  }
}

// Store a warp's 16 x (8*NT) accumulator as bf16 into a shared tile; `p` points at (m0, n0).
template <int NT>
__device__ __forceinline__ void acc_to_smem(__nv_bfloat16* p, int ld, const float (&acc)[NT][4], int lane) {
  int g = lane >> 2, t = lane & 3;
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    *reinterpret_cast<uint32_t*>(p + g * ld + nt * 8 + 2 * t) = pack_bf16(acc[nt][0], acc[nt][1]);
    *reinterpret_cast<uint32_t*>(p + (g + 8) * ld + nt * 8 + 2 * t) = pack_bf16(acc[nt][2], acc[nt][3]);
  }
}

template <int NT>
__device__ __forceinline__ void zero_acc(float (&acc)[NT][4]) {
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
  }
}

// Row-wise dot of a warp's accumulator with a bf16 shared tile at the same coordinates:
// r_lo = sum_n acc(g, n) * T(g, n), r_hi for row g+8; complete after the quad reduction.
template <int NT>
__device__ __forceinline__ void row_dot(float& r_lo, float& r_hi, const float (&acc)[NT][4], const __nv_bfloat16* p,
                                        int ld, int lane) {
  int g = lane >> 2, t = lane & 3;
  float lo = 0.f, hi = 0.f;
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    float2 a = unpack_bf16(*reinterpret_cast<const uint32_t*>(p + g * ld + nt * 8 + 2 * t));
    float2 b = unpack_bf16(*reinterpret_cast<const uint32_t*>(p + (g + 8) * ld + nt * 8 + 2 * t));
    lo += acc[nt][0] * a.x + acc[nt][1] * a.y;
    hi += acc[nt][2] * b.x + acc[nt][3] * b.y;
  }
  lo += __shfl_xor_sync(0xffffffffu, lo, 1);
  lo += __shfl_xor_sync(0xffffffffu, lo, 2);
  hi += __shfl_xor_sync(0xffffffffu, hi, 1);
  hi += __shfl_xor_sync(0xffffffffu, hi, 2);
  r_lo = lo;
  r_hi = hi;
}

// gamma is stored per chunk, [n_chunks][HV][64] fp32, entries past the chunk's valid length repeating the
// last valid value (so 2^(gamma_last - gamma_i) is 1 there): a chunk's 64 values are 256 contiguous,
// 256-byte aligned bytes that one bulk copy or one coalesced load brings in.
__device__ __forceinline__ const float* gamma_ptr(const float* gamma, int c, int HV, int hv) {
  return gamma + ((int64_t)c * HV + hv) * BT;
}
__device__ __forceinline__ void load_gamma(float* gs, const float* gamma, int c, int HV, int hv, int tid) {
  if (tid < BT) gs[tid] = gamma_ptr(gamma, c, HV, hv)[tid];
}
// Same through the async-copy path, so that the loading threads do not stall on the global latency.
__device__ __forceinline__ void load_gamma_async(float* gs, const float* gamma, int c, int HV, int hv, int tid) {
  if (tid < BT) cp_async4(gs + tid, gamma_ptr(gamma, c, HV, hv) + tid);
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
int launch_out_fwd(const b200gdn_chunk_args& a, cudaStream_t st);
int launch_dv_local(const b200gdn_chunk_args& a, cudaStream_t st);
int launch_scan_bwd(const b200gdn_chunk_args& a, cudaStream_t st);
int launch_bwd_dqk(const b200gdn_chunk_args& a, cudaStream_t st);
int launch_bwd_wy(const b200gdn_chunk_args& a, cudaStream_t st);
int launch_recurrent(const b200gdn_recurrent_args& a, cudaStream_t st);
int launch_affine(const b200gdn_affine_args& a, cudaStream_t st);
int launch_prep(const b200gdn_prep_args& a, cudaStream_t st, bool bwd);
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
