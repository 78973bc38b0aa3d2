// Tile-level helpers on top of tc5.cuh: swizzled staging of bf16 tiles, MMA issue loops over the
// contraction dimension, and accumulator read-back in the mma-fragment layout.
#pragma once
#include "gdn_common.cuh"
#include "tc5.cuh"

namespace gdn {

// ---- swizzled shared tile -> global ------------------------------------------------------------------------
// [ROWS][COLS] bf16 tile stored as 64-column panels of ROWS*128 bytes, 16-byte chunks XOR-swizzled with (row & 7);
// 16 bytes per access, rows < valid only (the ragged-chunk path; full chunks leave through TMA stores).
template <int ROWS, int COLS, int NTHREADS>
__device__ __forceinline__ void store_tile_swz(__nv_bfloat16* dst, int64_t gstride, const unsigned char* src, int valid,
                                               int tid) {
  constexpr int CPR = COLS / 8;
  constexpr int TOTAL = ROWS * CPR;
  static_assert(TOTAL % NTHREADS == 0, "tile/threads mismatch");
#pragma unroll
  for (int it = 0; it < TOTAL / NTHREADS; ++it) {
    int idx = it * NTHREADS + tid;
    int r = idx / CPR, c = idx % CPR;
    if (r < valid) {
      uint4 val = *reinterpret_cast<const uint4*>(src + (c >> 3) * (ROWS * 128) + r * 128 + (((c & 7) ^ (r & 7)) << 4));
      *reinterpret_cast<uint4*>(dst + (int64_t)r * gstride + c * 8) = val;
    }
  }
}

// 2^x with one MUFU instruction (ex2.approx.ftz: about 2 ulp, results below 2^-126 flush to zero).  The gate factors
// of this path are 2^(gamma_i - gamma_j) <= 1 multiplied into bf16-rounded tiles, so neither matters.
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}

// One 16-row x 32-column block of bf16 pairs in the accumulator-fragment layout (what acc_ld32 / acc_ld32q return,
// after the epilogue math) on its way into a swizzled tile: set() packs n-tile i, store() writes the block with two
// stmatrix.x4 (each moves eight rows of four 8 x 8 matrices; lane L supplies the address of row L % 8 of matrix L / 8),
// instead of eight 32-bit stores per thread.
struct FragStore {
  uint32_t lo[4], hi[4];
  __device__ __forceinline__ void set(int i, float a, float b, float c, float d) {
    lo[i] = pack_bf16(a, b);
    hi[i] = pack_bf16(c, d);
  }
  // rows row0 .. row0+15, columns col0 .. col0+31 (col0 a multiple of 8) of a tile of `rows` rows
  __device__ __forceinline__ void store(unsigned char* tile, int rows, int row0, int col0, int lane) const {
    store(tc5::smem_addr(tile), rows, row0, col0, lane);
  }
  // the same with the tile given by its shared-memory address
  __device__ __forceinline__ void store(uint32_t tile, int rows, int row0, int col0, int lane) const {
    const uint32_t addr = tile + tc5::swz_offset(row0 + (lane & 7), col0 + 8 * (lane >> 3), rows);
    asm volatile("stmatrix.sync.aligned.m8n8.x4.shared.b16 [%0], {%1, %2, %3, %4};\n" ::"r"(addr), "r"(lo[0]), "r"(lo[1]),
                 "r"(lo[2]), "r"(lo[3])
                 : "memory");
    asm volatile("stmatrix.sync.aligned.m8n8.x4.shared.b16 [%0], {%1, %2, %3, %4};\n" ::"r"(addr + 1024u), "r"(hi[0]),
                 "r"(hi[1]), "r"(hi[2]), "r"(hi[3])
                 : "memory");
  }
};

// The reverse: one 16-row x 32-column block of a swizzled bf16 tile into the accumulator-fragment layout with two
// ldmatrix.x4: lo[i] / hi[i] hold (row g, row g + 8) x columns (8 i + 2 t, + 1) of the block as bf16 pairs.
struct FragLoad {
  uint32_t lo[4], hi[4];
  __device__ __forceinline__ void load(uint32_t tile, int rows, int row0, int col0, int lane) {
    const uint32_t addr = tile + tc5::swz_offset(row0 + (lane & 7), col0 + 8 * (lane >> 3), rows);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];\n"
                 : "=r"(lo[0]), "=r"(lo[1]), "=r"(lo[2]), "=r"(lo[3])
                 : "r"(addr)
                 : "memory");
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];\n"
                 : "=r"(hi[0]), "=r"(hi[1]), "=r"(hi[2]), "=r"(hi[3])
                 : "r"(addr + 1024u)
                 : "memory");
  }
  __device__ __forceinline__ void load(const unsigned char* tile, int rows, int row0, int col0, int lane) {
    load(tc5::smem_addr(tile), rows, row0, col0, lane);
  }
  __device__ __forceinline__ float2 lo2(int i) const { return unpack_bf16(lo[i]); }
  __device__ __forceinline__ float2 hi2(int i) const { return unpack_bf16(hi[i]); }
};

// Zero rows [valid, ROWS) of a swizzled [ROWS][COLS] tile (a ragged last chunk arrives by TMA as a full box
// whose extra rows belong to the next sequence).  The caller fences and synchronises afterwards.
template <int ROWS, int COLS>
__device__ __forceinline__ void zero_tail_rows(unsigned char* tile, int valid, int tid, int nthreads) {
  constexpr int CPR = COLS / 8;
  const int total = (ROWS - valid) * CPR;
  for (int idx = tid; idx < total; idx += nthreads) {
    const int r = valid + idx / CPR, c = idx % CPR;
    *reinterpret_cast<uint4*>(tile + (c >> 3) * (ROWS * 128) + r * 128 + (((c & 7) ^ (r & 7)) << 4)) = make_uint4(0, 0, 0, 0);
  }
}

// ---- MMA issue (one thread) -----------------------------------------------------------------------------
// Operand descriptions.  A tile is stored [rows][cols]; as a K-major operand its MN index runs over rows
// and the contraction over columns; as an MN-major operand the MN index runs over columns and the
// contraction over rows.
struct Operand {
  uint32_t saddr;   // shared address of the tile (1024-byte aligned) plus any panel offset
  int rows;         // rows of the stored tile (panel stride = rows * 128 bytes)
  int mn_major;     // 0: K-major, 1: MN-major
};
__device__ __forceinline__ uint64_t operand_desc0(const Operand& o) {
  return o.mn_major ? tc5::smem_desc(o.saddr, o.rows * 128, 1024) : tc5::smem_desc(o.saddr, 16, 1024);
}
// byte offset of contraction step `kstep` (16 elements) from the operand's first descriptor
__device__ __forceinline__ uint32_t operand_step_bytes(const Operand& o, int kstep) {
  return o.mn_major ? (uint32_t)kstep * 2048u : (uint32_t)((kstep >> 2) * o.rows * 128 + (kstep & 3) * 32);
}
// D[tmem] (+)= A B over KSTEPS steps of 16.  `acc` = 0 starts a fresh accumulator.  The two base descriptors
// are built once; every step only adds its byte offset (>> 4) to the address field.
template <int KSTEPS>
__device__ __forceinline__ void issue_mma_t(uint32_t d_tmem, const Operand& a, const Operand& b, int M, int N, int acc,
                                            int neg_a = 0) {
  const uint32_t idesc = tc5::idesc_bf16(M, N, a.mn_major, b.mn_major, neg_a);
  const uint64_t da = operand_desc0(a), db = operand_desc0(b);
#pragma unroll
  for (int ks = 0; ks < KSTEPS; ++ks)
    tc5::mma_ss(d_tmem, da + (operand_step_bytes(a, ks) >> 4), db + (operand_step_bytes(b, ks) >> 4), idesc,
                (acc || ks > 0) ? 1u : 0u);
}
// ---- accumulator read-back -------------------------------------------------------------------------------
// 16 rows x 32 columns of an M = 64 accumulator for this warp (rows 16*warp .. +15): r[4*i + e] is
// n-tile i (columns c0 + 8i ..), e = {row g col 2t, row g col 2t+1, row g+8 col 2t, row g+8 col 2t+1}.
__device__ __forceinline__ void acc_ld32(uint32_t tmem_acc, int warp, int c0, float (&r)[16]) {
  tc5::tmem_ld_16x256b_x4(tmem_acc + ((uint32_t)(warp * 32) << 16) + c0, r);
}

// The same block for a CTA of eight warps: warps w and w + 4 share TMEM quadrant w & 3 and split the
// columns, `c0` is relative to the warp's own half.
__device__ __forceinline__ void acc_ld32q(uint32_t tmem_acc, int quad, int c0, float (&r)[16]) {
  tc5::tmem_ld_16x256b_x4(tmem_acc + ((uint32_t)(quad * 32) << 16) + c0, r);
}

// One phase boundary: the issuing thread commits, everybody waits for the MMAs (bounded).
struct PhaseBarrier {
  uint64_t* bar;
  uint32_t parity;
  int* err;
  __device__ __forceinline__ void commit() { tc5::mma_commit(bar); }
  __device__ __forceinline__ bool wait() {
    bool ok = tc5::mbar_wait(bar, parity);
    parity ^= 1u;
    tc5::fence_after_sync();
    return ok;
  }
  // CTA-wide form: the first warp polls the barrier, the others sleep in the hardware barrier instead of
  // spending issue slots on the poll; returns false if the wait expired or any thread passed `bad`.
  // (Pays in kernels whose other resident CTAs are issue-bound; measured slower in the two big backward kernels.)
  __device__ __forceinline__ bool sync_wait(bool bad = false) {
    if (threadIdx.x < 32 && !bad) bad = !tc5::mbar_wait(bar, parity);
    parity ^= 1u;
    const int any_bad = __syncthreads_or(bad);
    tc5::fence_after_sync();
    return !any_bad;
  }
};

}  // namespace gdn
