// tcgen05 / TMEM / mbarrier primitives for sm_100a (inline PTX), used by the chunk-parallel kernels.
//
// Conventions
//  * one CTA, cta_group::1; accumulators live in tensor memory (TMEM: 128 lanes x 512 32-bit columns);
//  * operands are bf16 tiles in shared memory in the canonical 128-byte-swizzled layout: a tile is a
//    stack of "panels" of 64 columns (128 bytes) per row; inside each group of 8 rows (1024 bytes) the
//    16-byte chunk index is XORed with the row index (what TMA's SWIZZLE_128B writes).  The same bytes
//    serve as a K-major operand (MN = rows, K = columns) or as an MN-major operand (MN = columns,
//    K = rows), which is how transposed products are issued without moving data;
//  * an M = 64 accumulator occupies lanes 0-15 of each of the four 32-lane quadrants (row r -> lane
//    32*(r/16) + r%16); an M = 128 accumulator occupies lane r;
//  * every wait is bounded: on expiry the caller sets an error flag and leaves.
#pragma once
#include <cuda_bf16.h>
#include <stdint.h>

namespace tc5 {

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

// ---- mbarrier ------------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_addr(bar)), "r"(count));
}
__device__ __forceinline__ void fence_mbar_init() { asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory"); }
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_addr(bar)) : "memory");
}
// Bounded wait for the phase with the given parity.  Returns false when the limit expires.
// (A legitimate wait in these kernels lasts microseconds; the default limit is seconds of polling.)
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, uint32_t limit = (1u << 22)) {
  const uint32_t addr = smem_addr(bar);
  for (uint32_t it = 0; it < limit; ++it) {
    uint32_t done;
    asm volatile(
        "{\n.reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(done)
        : "r"(addr), "r"(parity)
        : "memory");
    if (done) return true;
  }
  return false;
}

// generic-proxy writes to shared memory -> visible to the async proxy (tensor core / TMA reads)
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory"); }

// ---- tensor memory -------------------------------------------------------------------------------------
// Executed by one full warp.  `slot` (shared memory) receives the base address (lane 0, first column).
__device__ __forceinline__ void tmem_alloc(uint32_t* slot, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_addr(slot)), "r"(ncols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }

// ---- descriptors ---------------------------------------------------------------------------------------
// Shared-memory matrix descriptor, 128-byte swizzle (layout type 2), descriptor version 1.
//   K-major : lbo = 1 (unused), sbo = bytes between 8-row groups (1024 for a dense panel)
//   MN-major: lbo = bytes between 64-column panels, sbo = bytes between 8-row groups (1024)
__device__ __forceinline__ uint64_t smem_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr >> 4) & 0x3FFFu);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= 1ull << 46;   // version
  d |= 2ull << 61;   // SWIZZLE_128B
  return d;
}

// Instruction descriptor for kind::f16 with bf16 operands and fp32 accumulation.
//   a_mn / b_mn : operand is MN-major (1) or K-major (0);  neg_a: D -= A B instead of +=
__host__ __device__ constexpr uint32_t idesc_bf16(int M, int N, int a_mn, int b_mn, int neg_a = 0) {
  return (1u << 4)                    // D format fp32
         | (1u << 7) | (1u << 10)     // A, B format bf16
         | ((uint32_t)neg_a << 13) | ((uint32_t)a_mn << 15) | ((uint32_t)b_mn << 16) | ((uint32_t)(N >> 3) << 17) |
         ((uint32_t)(M >> 4) << 24);
}

// D[tmem] (+)= A[smem] B[smem]; issued by ONE thread.
__device__ __forceinline__ void mma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// All previously issued MMAs of this thread arrive on `bar` when they complete.
__device__ __forceinline__ void mma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(smem_addr(bar))
               : "memory");
}

// ---- TMEM -> registers -------------------------------------------------------------------------------
// 16 lanes x 256 bits per repetition: thread t of the warp receives, for each group of 8 columns,
// (row t/4, cols 2(t%4), 2(t%4)+1) in r[4i+0..1] and (row t/4 + 8, same cols) in r[4i+2..3] - the
// accumulator-fragment layout of mma.sync m16n8.  `taddr` = base + (first lane << 16) + first column.
__device__ __forceinline__ void tmem_ld_16x256b_x4(uint32_t taddr, float (&r)[16]) {
  uint32_t* u = reinterpret_cast<uint32_t*>(r);
  asm volatile(
      "tcgen05.ld.sync.aligned.16x256b.x4.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n"
      : "=r"(u[0]), "=r"(u[1]), "=r"(u[2]), "=r"(u[3]), "=r"(u[4]), "=r"(u[5]), "=r"(u[6]), "=r"(u[7]), "=r"(u[8]),
        "=r"(u[9]), "=r"(u[10]), "=r"(u[11]), "=r"(u[12]), "=r"(u[13]), "=r"(u[14]), "=r"(u[15])
      : "r"(taddr));
}
// registers -> TMEM, same element mapping as tmem_ld_16x256b_x4
__device__ __forceinline__ void tmem_st_16x256b_x4(uint32_t taddr, const float (&r)[16]) {
  const uint32_t* u = reinterpret_cast<const uint32_t*>(r);
  asm volatile(
      "tcgen05.st.sync.aligned.16x256b.x4.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};\n" ::"r"(taddr),
      "r"(u[0]), "r"(u[1]), "r"(u[2]), "r"(u[3]), "r"(u[4]), "r"(u[5]), "r"(u[6]), "r"(u[7]), "r"(u[8]), "r"(u[9]), "r"(u[10]),
      "r"(u[11]), "r"(u[12]), "r"(u[13]), "r"(u[14]), "r"(u[15])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory"); }
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }

// ---- swizzled shared tiles ---------------------------------------------------------------------------
// Byte offset of element (row, col) in a tile of `rows` rows stored as 64-column panels with the
// 128-byte swizzle.  The tile base must be 1024-byte aligned.
__device__ __forceinline__ uint32_t swz_offset(int row, int col, int rows) {
  int panel = col >> 6, c = col & 63;
  return (uint32_t)(panel * rows * 128 + row * 128 + ((((c >> 3) ^ (row & 7)) << 4) | ((c & 7) << 1)));
}

}  // namespace tc5
