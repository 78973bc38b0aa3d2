// Backward of the WY representation on tcgen05 tensor cores with TMEM accumulators, fused with
// dw = -dv2 h^T (so dw never touches HBM), the final sum of dk and the reverse chunk-local cumsum of dg.
// Replaces prepare_wy_repr_bwd_kernel (fla/ops/gated_delta_rule/wy_fast.py:123-251), the dw part of
// chunk_bwd_kernel_dqkwg (fla/ops/common/chunk_o.py:246-260) and chunk.py:244-246 of the reference.
//
//     dW   = -dU h^T                                    dU = dv2
//     dA   = strict_tril((dW K^T) (beta 2^gamma)_j + (dU V^T) beta_j)
//     M    = -strict_tril(A^T dA A^T) 2^(gamma_i - gamma_j),   M2 = M beta_i
//     dk   = (chunk-local part from the dq/dk kernel) + (A beta 2^gamma)_col^T dW + M2 K + M2^T K
//     dv   = (A^T dU) beta_i
//     dbeta= colsum(A . dW K^T) 2^gamma + colsum(A . dU V^T) + rowsum(M . K K^T)
//     dG   = dG_part + colsum(A . dW K^T) beta 2^gamma + beta rowsum(M . K K^T) - colsum(M2 . K K^T)
//     dg   = reverse cumsum of dG inside the chunk
// All row scalings are folded into operands and all 128-wide row-dots are replaced by sums over 64x64
// tiles that exist anyway (dW K^T, dU V^T, K K^T), so the three dk terms accumulate in one TMEM tile.
//
// One CTA of eight warps per (chunk, q/k head).  The epilogues between the five dependent MMA phases are
// CUDA-core work on 64-row tiles, so they are spread over eight warps (warps w and w+4 share TMEM
// quadrant w&3 and split the columns); all tiles arrive by TMA issued from one thread.  256 TMEM columns
// and ~100 KiB of shared memory: two CTAs per SM overlap each other's phases.
#include "tc5_tile.cuh"
#include "tma.cuh"

namespace gdn {
namespace {

constexpr int NTHREADS = 256;
__device__ int g_wy_timeout = 0;

template <int DK, int DV>
struct WyTcSmem {
  static constexpr size_t o_k = 0;
  static constexpr size_t o_v = o_k + BT * DK * 2;     // V; later dA (8 KiB) | Y (8 KiB)
  static constexpr size_t v_bytes = BT * DV * 2 > 2 * BT * 128 ? BT * DV * 2 : 2 * BT * 128;
  static constexpr size_t o_du = o_v + v_bytes;
  static constexpr size_t o_a = o_du + BT * DV * 2;    // A
  static constexpr size_t o_ab = o_a + BT * 128;       // A (beta 2^gamma)_col
  static constexpr size_t o_h = o_ab + BT * 128;       // h [DK][DV]; later dW (BT*DK*2) | dv staging / M2
  static constexpr size_t h_bytes = DK * DV * 2 > BT * DK * 2 + BT * DV * 2 ? DK * DV * 2 : BT * DK * 2 + BT * DV * 2;
  static constexpr size_t o_vec = o_h + h_bytes;
  static constexpr size_t bytes = o_vec + 6144 + 1024;
};

struct WyMaps {
  CUtensorMap k, v, du, a, h, dv, dk;
};

// Eight values per lane (v[2 i + p]: n-tile i, column parity p), each to be summed over the eight row-lanes of the warp
// (lanes that differ in bits 2..4).  Recursive halving: 7 shuffles instead of 24; afterwards the lane with row index g
// holds the complete sum of value g, i.e. of column 8 (g >> 1) + 2 t + (g & 1) of the warp's 32-column block.
__device__ __forceinline__ float sum8_over_g(const float (&v)[8], int g) {
  float w[4], x[2];
  const bool h4 = g & 4, h2 = g & 2, h1 = g & 1;
#pragma unroll
  for (int j = 0; j < 4; ++j) w[j] = (h4 ? v[4 + j] : v[j]) + __shfl_xor_sync(0xffffffffu, h4 ? v[j] : v[4 + j], 16);
#pragma unroll
  for (int j = 0; j < 2; ++j) x[j] = (h2 ? w[2 + j] : w[j]) + __shfl_xor_sync(0xffffffffu, h2 ? w[j] : w[2 + j], 8);
  return (h1 ? x[1] : x[0]) + __shfl_xor_sync(0xffffffffu, h1 ? x[0] : x[1], 4);
}
__device__ __forceinline__ float sum_over_t(float x) {
  x += __shfl_xor_sync(0xffffffffu, x, 1);
  x += __shfl_xor_sync(0xffffffffu, x, 2);
  return x;
}

// GROUPED: more than one value head per q/k head (the heads of a group are walked by one CTA and their dk terms
// add up in fp32 through dk_part); the common ungrouped case is compiled without that path.
template <int DK, int DV, bool GROUPED>
__global__ void __launch_bounds__(NTHREADS, 2) bwd_wy_kernel(const b200gdn_chunk_args a, const __grid_constant__ WyMaps maps) {
  using S = WyTcSmem<DK, DV>;
  constexpr int KB = DK / 64, VB = DV / 64;   // 32-column blocks of a wide accumulator per warp
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* Ks = smem + S::o_k;
  unsigned char* Vs = smem + S::o_v;
  unsigned char* dAs = smem + S::o_v;
  unsigned char* Ys = smem + S::o_v + BT * 128;
  unsigned char* dUs = smem + S::o_du;
  unsigned char* As = smem + S::o_a;
  unsigned char* Abs = smem + S::o_ab;
  unsigned char* Hs = smem + S::o_h;
  unsigned char* dWs = smem + S::o_h;
  unsigned char* Stg = smem + S::o_h + BT * DK * 2;   // dv staging, then M2
  unsigned char* M2s = Stg;
  float* gs = reinterpret_cast<float*>(smem + S::o_vec);
  float* bet = gs + BT;
  float* bge = bet + BT;
  float* eg = bge + BT;
  float* dGin = eg + BT;
  float* dGs = dGin + BT;
  // column sums are reduced over rows: each of the four row-quadrant warps leaves its partial in its own
  // slot and the consumer adds the four in a fixed order (no atomics: results are bit-reproducible)
  float* c_kbg = dGs + BT;       // [4][64] colsum(A . dW K^T)
  float* c_vb = c_kbg + 4 * BT;  // [4][64] colsum(A . dU V^T)
  float* c_m2 = c_vb + 4 * BT;   // [4][64] colsum(M2 . K K^T)
  float* r_mk = c_m2 + 4 * BT;   // rowsum(M . K K^T), two column halves
  float* sgm = r_mk + 2 * BT;    // fused beta option: sigmoid(raw beta), for its derivative
  float* gx = sgm + BT;          // fused gate option: raw g + dt_bias
  float* gred = gx + BT;         // [4] partial sums of the gate-parameter gradients (two warps)
  uint64_t* bar = reinterpret_cast<uint64_t*>(gred + 4);
  uint64_t* bar_ld = bar + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_ld + 1);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int q = warp & 3, hc = warp >> 2;
  const int g = lane >> 2, t = lane & 3;
  const int c = blockIdx.x, hq = blockIdx.y;
  const int G = GROUPED ? a.HV / a.H : 1;
  const ChunkMeta cm = load_chunk_meta(a.chunk_meta, c);
  const int64_t row0 = cm.row;
  const int r_lo = q * 16 + g, r_hi = r_lo + 8;
  const int cs = hc * 32;   // this warp's 32 columns of a 64-column tile

  auto issue_loads = [&](int gi) {   // one thread
    const int hv = hq * G + gi;
    const uint32_t tx = (uint32_t)((gi == 0 ? BT * DK * 2 : 0) + 2 * BT * DV * 2 + BT * 128 + DK * DV * 2 + BT * 4);
    tc5::mbar_expect_tx(bar_ld, tx);
    tma::load_3d(dUs, &maps.du, cm.row, (hv * DV) / 64, bar_ld);
    tma::load_3d(Hs, &maps.h, (c * a.HV + hv) * DK, 0, bar_ld);
    if (gi == 0) tma::load_3d(Ks, &maps.k, cm.row, (hq * DK) / 64, bar_ld);
    tma::load_3d(Vs, &maps.v, cm.row, (hv * DV) / 64, bar_ld);
    tma::load_2d(As, &maps.a, hv * BT, cm.row, bar_ld);
    tma::load_1d(gs, gamma_ptr(a.gamma, c, a.HV, hv), BT * 4, bar_ld);
  };
  if (tid == 0) {
    tc5::mbar_init(bar, 1);
    tc5::mbar_init(bar_ld, 1);
    tc5::fence_mbar_init();
    issue_loads(0);   // the first head's tiles are on their way while the CTA sets itself up
  }

  if (warp == 1) tc5::tmem_alloc(tmem_slot, 256);
  {
    // the dq/dk kernel's part of dk (bf16, in the dk buffer) is read at the very end: pull it into L2 now
    const int r = tid >> 2, seg = tid & 3;
    if (r < cm.len && seg * 64 < DK)
      tma::prefetch_line(reinterpret_cast<const __nv_bfloat16*>(a.dk) + ((row0 + r) * a.H + hq) * DK + seg * 64);

  }
  tc5::fence_before_sync();
  __syncthreads();
  tc5::fence_after_sync();
  const uint32_t tm = *tmem_slot;
  const uint32_t TM_BIG = tm, TM_S1 = tm + 128, TM_KK = tm + 192;   // 128 | 64 | 64 columns
  PhaseBarrier ph{bar, 0u, &g_wy_timeout};
  bool failed = false;

  const Operand opK_k{tc5::smem_addr(Ks), BT, 0};    // K as (n = token, k = key dim)
  const Operand opK_mn{tc5::smem_addr(Ks), BT, 1};   // K as (k = token, n = key dim)
  const Operand opA_k{tc5::smem_addr(As), BT, 0};    // A as (n = row j, k = col b)
  const Operand opA_mn{tc5::smem_addr(As), BT, 1};   // A^T : (m = col, k = row)
  const Operand opAb_mn{tc5::smem_addr(Abs), BT, 1};
  const Operand opdU_k{tc5::smem_addr(dUs), BT, 0};
  const Operand opdU_mn{tc5::smem_addr(dUs), BT, 1};
  const Operand opdW_k{tc5::smem_addr(dWs), BT, 0};
  const Operand opdW_mn{tc5::smem_addr(dWs), BT, 1};

  for (int gi = 0; gi < G && !failed; ++gi) {
    const int hv = hq * G + gi;
    const bool last = gi == G - 1;
    if (gi > 0) {
      __syncthreads();   // previous head fully consumed
      if (tid == 0) issue_loads(gi);
    }
    if (tid < BT) {
      const bool ok = tid < cm.len;
      float b = ok ? a.beta[(row0 + tid) * a.HV + hv] : 0.f;
      if (a.options & B200GDN_PREP_BETA_SIGMOID) {   // raw beta: the kernels work with (1|2) sigmoid(beta)
        const float sg = 1.f / (1.f + expf(-b));
        sgm[tid] = sg;
        b = ok ? ((a.options & B200GDN_PREP_NEG_EIGVAL) ? 2.f : 1.f) * sg : 0.f;
      }
      bet[tid] = b;
      if (a.options & B200GDN_PREP_GATE)
        gx[tid] = (ok ? a.g[(row0 + tid) * a.HV + hv] : 0.f) + (a.dt_bias ? a.dt_bias[hv] : 0.f);
      dGin[tid] = ok ? a.dG[(row0 + tid) * a.HV + hv] : 0.f;
    }
    if (!tc5::mbar_wait(bar_ld, gi & 1)) failed = true;
    if (cm.len < BT) {   // ragged chunk: the extra rows of the boxes belong to the next sequence
      if (gi == 0) zero_tail_rows<BT, DK>(Ks, cm.len, tid, NTHREADS);
      zero_tail_rows<BT, DV>(Vs, cm.len, tid, NTHREADS);
      zero_tail_rows<BT, DV>(dUs, cm.len, tid, NTHREADS);
      zero_tail_rows<BT, BT>(As, cm.len, tid, NTHREADS);
    }
    if (tid < BT) {   // bet[tid] was written by this very thread
      const float e = fast_exp2(gs[tid]);
      eg[tid] = e;
      bge[tid] = bet[tid] * e;
    }
    tc5::fence_async_smem();
    if (__syncthreads_or(failed)) { failed = true; break; }

    // ---- phase 1: dW = -dU h^T | dA2 = dU V^T | KK = K K^T
    if (tid == 0) {
      tc5::fence_after_sync();
      issue_mma_t<DV / 16>(TM_BIG, opdU_k, Operand{tc5::smem_addr(Hs), DK, 0}, 64, DK, 0, /*neg_a=*/1);
      issue_mma_t<DV / 16>(TM_S1, opdU_k, Operand{tc5::smem_addr(Vs), BT, 0}, 64, 64, 0);
      issue_mma_t<DK / 16>(TM_KK, opK_k, opK_k, 64, 64, 0);
      ph.commit();
    }
    // A with its columns scaled by beta 2^gamma (an operand of phase 3), while phase 1 runs
    {   // every warp rescales its own 16 x 32 block of the tile
      FragLoad fa;
      fa.load(As, BT, q * 16, cs, lane);
      FragStore fs;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 sc = *reinterpret_cast<const float2*>(&bge[cs + i * 8 + 2 * t]);
        const float2 al = fa.lo2(i), ah = fa.hi2(i);
        fs.set(i, al.x * sc.x, al.y * sc.y, ah.x * sc.x, ah.y * sc.y);
      }
      fs.store(Abs, BT, q * 16, cs, lane);
    }
    const float g_lo = gs[r_lo], g_hi = gs[r_hi];
    const float b_lo = bet[r_lo], b_hi = bet[r_hi];
    if (__syncthreads_or(!ph.wait())) { failed = true; break; }

    // ---- epilogue 1: dW -> shared (over the h buffer); dA2 -> registers; colsum(A . dA2)
    {
      float r[KB][16];
#pragma unroll
      for (int b = 0; b < KB; ++b) acc_ld32q(TM_BIG, q, hc * (DK / 2) + b * 32, r[b]);
      tc5::tmem_ld_wait();
#pragma unroll
      for (int b = 0; b < KB; ++b) {
        FragStore fs;
#pragma unroll
        for (int i = 0; i < 4; ++i) fs.set(i, r[b][4 * i], r[b][4 * i + 1], r[b][4 * i + 2], r[b][4 * i + 3]);
        fs.store(dWs, BT, q * 16, hc * (DK / 2) + b * 32, lane);
      }
    }
    float dA2[16];
    acc_ld32q(TM_S1, q, cs, dA2);
    tc5::tmem_ld_wait();
    tc5::fence_async_smem();
    tc5::fence_before_sync();
    __syncthreads();

    // ---- phase 2: dA1 = dW K^T | dVb = A^T dU
    if (tid == 0) {
      tc5::fence_after_sync();
      issue_mma_t<DK / 16>(TM_S1, opdW_k, opK_k, 64, 64, 0);
      issue_mma_t<BT / 16>(TM_BIG, opA_mn, opdU_mn, 64, DV, 0);
      ph.commit();
    }
    // colsum(A . dA2), off the critical path
    const int gcol = cs + 8 * (g >> 1) + 2 * t + (g & 1);   // the column whose sum this lane ends up with
    {
      FragLoad fa;
      fa.load(As, BT, q * 16, cs, lane);
      float pv[8];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 al = fa.lo2(i), ah = fa.hi2(i);
        pv[2 * i] = al.x * dA2[4 * i] + ah.x * dA2[4 * i + 2];
        pv[2 * i + 1] = al.y * dA2[4 * i + 1] + ah.y * dA2[4 * i + 3];
      }
      c_vb[q * BT + gcol] = sum8_over_g(pv, g);
    }
    if (__syncthreads_or(!ph.wait())) { failed = true; break; }

    // ---- epilogue 2: dA -> shared (over V) is all phase 3 waits for; colsum(A . dA1) and dv = dVb beta follow
    {
      float r[16];
      acc_ld32q(TM_S1, q, cs, r);
      float rv[VB][16];
#pragma unroll
      for (int b = 0; b < VB; ++b) acc_ld32q(TM_BIG, q, hc * (DV / 2) + b * 32, rv[b]);
      tc5::tmem_ld_wait();
      FragStore fs_dA;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int col = cs + i * 8 + 2 * t;
        float v[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int ii = (e & 2) ? r_hi : r_lo, jj = col + (e & 1);
          v[e] = (ii > jj) ? r[4 * i + e] * bge[jj] + dA2[4 * i + e] * bet[jj] : 0.f;
        }
        fs_dA.set(i, v[0], v[1], v[2], v[3]);
      }
      fs_dA.store(dAs, BT, q * 16, cs, lane);
      tc5::fence_async_smem();
      tc5::fence_before_sync();
      __syncthreads();

      // ---- phase 3: Y = dA A^T | dk = (A beta 2^gamma)^T dW
      if (tid == 0) {
        tc5::fence_after_sync();
        issue_mma_t<BT / 16>(TM_S1, Operand{tc5::smem_addr(dAs), BT, 0}, opA_k, 64, 64, 0);
        issue_mma_t<BT / 16>(TM_BIG, opAb_mn, opdW_mn, 64, DK, 0);
        ph.commit();
      }
      {
        FragLoad fa;
        fa.load(As, BT, q * 16, cs, lane);
        float pv[8];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 al = fa.lo2(i), ah = fa.hi2(i);
          pv[2 * i] = al.x * r[4 * i] + ah.x * r[4 * i + 2];
          pv[2 * i + 1] = al.y * r[4 * i + 1] + ah.y * r[4 * i + 3];
        }
        c_kbg[q * BT + gcol] = sum8_over_g(pv, g);
      }
#pragma unroll
      for (int b = 0; b < VB; ++b) {
        FragStore fs;
#pragma unroll
        for (int i = 0; i < 4; ++i)
          fs.set(i, rv[b][4 * i] * b_lo, rv[b][4 * i + 1] * b_lo, rv[b][4 * i + 2] * b_hi, rv[b][4 * i + 3] * b_hi);
        fs.store(Stg, BT, q * 16, hc * (DV / 2) + b * 32, lane);
      }
    }
    tc5::fence_async_smem();
    __syncthreads();
    if (cm.len == BT) {
      if (tid == 32) {
        tma::store_3d(&maps.dv, (int)cm.row, (hv * DV) / 64, Stg);
        tma::store_commit();
      }
    } else {
      store_tile_swz<BT, DV, NTHREADS>(reinterpret_cast<__nv_bfloat16*>(a.dv) + (row0 * a.HV + hv) * DV, (int64_t)a.HV * DV,
                                       Stg, cm.len, tid);
    }
    if (__syncthreads_or(!ph.wait())) { failed = true; break; }

    // ---- epilogue 3: Y -> shared
    {
      float r[16];
      acc_ld32q(TM_S1, q, cs, r);
      tc5::tmem_ld_wait();
      FragStore fs;
#pragma unroll
      for (int i = 0; i < 4; ++i) fs.set(i, r[4 * i], r[4 * i + 1], r[4 * i + 2], r[4 * i + 3]);
      fs.store(Ys, BT, q * 16, cs, lane);
    }
    if (tid == 32) tma::store_wait_read<0>();   // the dv staging tile is rewritten (as M2) after the next barrier
    tc5::fence_async_smem();
    tc5::fence_before_sync();
    __syncthreads();

    // ---- phase 4: X = A^T Y
    if (tid == 0) {
      tc5::fence_after_sync();
      issue_mma_t<BT / 16>(TM_S1, opA_mn, Operand{tc5::smem_addr(Ys), BT, 1}, 64, 64, 0);
      ph.commit();
    }
    if (__syncthreads_or(!ph.wait())) { failed = true; break; }

    // ---- epilogue 4: M2 = M beta_i -> shared is all phase 5 waits for; the sums over M . KK follow
    float m[16], kk[16];
    {
      float r[16];
      acc_ld32q(TM_S1, q, cs, r);
      acc_ld32q(TM_KK, q, cs, kk);
      tc5::tmem_ld_wait();
      FragStore fs_m2;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int col = cs + i * 8 + 2 * t;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int ii = (e & 2) ? r_hi : r_lo, jj = col + (e & 1);
          m[4 * i + e] = (ii > jj) ? -r[4 * i + e] * fast_exp2(((e & 2) ? g_hi : g_lo) - gs[jj]) : 0.f;
        }
        fs_m2.set(i, m[4 * i] * b_lo, m[4 * i + 1] * b_lo, m[4 * i + 2] * b_hi, m[4 * i + 3] * b_hi);
      }
      fs_m2.store(M2s, BT, q * 16, cs, lane);
    }
    tc5::fence_async_smem();
    tc5::fence_before_sync();
    __syncthreads();

    // ---- phase 5: dk += M2 K + M2^T K
    if (tid == 0) {
      tc5::fence_after_sync();
      issue_mma_t<BT / 16>(TM_BIG, Operand{tc5::smem_addr(M2s), BT, 0}, opK_mn, 64, DK, 1);
      issue_mma_t<BT / 16>(TM_BIG, Operand{tc5::smem_addr(M2s), BT, 1}, opK_mn, 64, DK, 1);
      ph.commit();
    }
    {
      float rmk_lo = 0.f, rmk_hi = 0.f;
      float pv[8];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        rmk_lo += m[4 * i] * kk[4 * i] + m[4 * i + 1] * kk[4 * i + 1];
        rmk_hi += m[4 * i + 2] * kk[4 * i + 2] + m[4 * i + 3] * kk[4 * i + 3];
        pv[2 * i] = m[4 * i] * b_lo * kk[4 * i] + m[4 * i + 2] * b_hi * kk[4 * i + 2];
        pv[2 * i + 1] = m[4 * i + 1] * b_lo * kk[4 * i + 1] + m[4 * i + 3] * b_hi * kk[4 * i + 3];
      }
      c_m2[q * BT + gcol] = sum8_over_g(pv, g);
      rmk_lo = sum_over_t(rmk_lo);
      rmk_hi = sum_over_t(rmk_hi);
      if (t == 0) {
        r_mk[hc * BT + r_lo] = rmk_lo;
        r_mk[hc * BT + r_hi] = rmk_hi;
      }
    }
    // the dq/dk kernel's part of dk: fetched now so that its latency hides behind the MMAs
    float* const dkbuf = a.dk_part + (row0 * a.H + hq) * DK + hc * (DK / 2);
    const int64_t dkstride = (int64_t)a.H * DK;
    // first head of the group: the bf16 sum the dq/dk kernel left in the dk buffer; later heads: the fp32 running
    // sum of this kernel (dk_part)
    const __nv_bfloat16* const dkin = reinterpret_cast<const __nv_bfloat16*>(a.dk) + (row0 * a.H + hq) * DK + hc * (DK / 2);
    uint32_t part16[GROUPED ? 1 : KB * 4][2];        // ungrouped: bf16 pairs, unpacked when they are used
    float2 part32[GROUPED ? KB * 4 : 1][2];          // grouped: fp32 pairs
#pragma unroll
    for (int n8 = 0; n8 < KB * 4; ++n8) {
      const int col = n8 * 8 + 2 * t;
      if (!GROUPED) {
        part16[n8][0] = r_lo < cm.len ? *reinterpret_cast<const uint32_t*>(dkin + r_lo * dkstride + col) : 0u;
        part16[n8][1] = r_hi < cm.len ? *reinterpret_cast<const uint32_t*>(dkin + r_hi * dkstride + col) : 0u;
      } else if (gi == 0) {
        part32[n8][0] = unpack_bf16(r_lo < cm.len ? *reinterpret_cast<const uint32_t*>(dkin + r_lo * dkstride + col) : 0u);
        part32[n8][1] = unpack_bf16(r_hi < cm.len ? *reinterpret_cast<const uint32_t*>(dkin + r_hi * dkstride + col) : 0u);
      } else {
        part32[n8][0] = r_lo < cm.len ? *reinterpret_cast<const float2*>(dkbuf + r_lo * dkstride + col) : make_float2(0.f, 0.f);
        part32[n8][1] = r_hi < cm.len ? *reinterpret_cast<const float2*>(dkbuf + r_hi * dkstride + col) : make_float2(0.f, 0.f);
      }
    }
    __syncthreads();   // column / row sums of every warp are in place
    // gate / beta gradients while the MMAs run: dG per row, then the reverse cumsum as a two-warp suffix scan
    if (tid < BT) {
      const int i = tid;
      const float rmk = r_mk[i] + r_mk[BT + i];
      const float ckbg = (c_kbg[i] + c_kbg[BT + i]) + (c_kbg[2 * BT + i] + c_kbg[3 * BT + i]);
      const float cvb = (c_vb[i] + c_vb[BT + i]) + (c_vb[2 * BT + i] + c_vb[3 * BT + i]);
      const float cm2 = (c_m2[i] + c_m2[BT + i]) + (c_m2[2 * BT + i] + c_m2[3 * BT + i]);
      float x = ckbg * bge[i] + bet[i] * rmk - cm2 + dGin[i];
      if (i < cm.len) {
        float db = ckbg * eg[i] + cvb + rmk;
        if (a.options & B200GDN_PREP_BETA_SIGMOID)   // chain rule through (1|2) sigmoid
          db *= ((a.options & B200GDN_PREP_NEG_EIGVAL) ? 2.f : 1.f) * sgm[i] * (1.f - sgm[i]);
        a.dbeta[(row0 + i) * a.HV + hv] = db;
      }
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const float y = __shfl_down_sync(0xffffffffu, x, o);
        if (lane + o < 32) x += y;
      }
      dGs[i] = x;   // suffix sum inside the warp
    }
    if (__syncthreads_or(!ph.wait())) { failed = true; break; }
    if (!(a.options & B200GDN_PREP_GATE)) {
      if (tid < cm.len) a.dg[(row0 + tid) * a.HV + hv] = dGs[tid] + (tid < 32 ? dGs[32] : 0.f);
    } else {
      // fused gate: g = -exp(A_log) softplus(x), x = g_raw + dt_bias.  dg_raw = dg (-exp(A_log)) sigmoid(x);
      // dA_log += dg g and ddt_bias += dg_raw, summed over the chunk here and over the chunks by a second kernel
      if (tid < BT) {
        float sA = 0.f, sB = 0.f;
        if (tid < cm.len) {
          const float dgi = dGs[tid] + (tid < 32 ? dGs[32] : 0.f);
          const float x = gx[tid], negA = -expf(a.A_log[hv]);
          const float draw = dgi * negA / (1.f + expf(-x));
          a.dg[(row0 + tid) * a.HV + hv] = draw;
          sA = dgi * negA * (x > 20.f ? x : log1pf(expf(x)));
          sB = draw;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
          sA += __shfl_xor_sync(0xffffffffu, sA, o);
          sB += __shfl_xor_sync(0xffffffffu, sB, o);
        }
        if (lane == 0) {
          gred[2 * warp] = sA;
          gred[2 * warp + 1] = sB;
        }
      }
      __syncthreads();
      if (tid == 0) {
        a.gate_partials[((int64_t)c * a.HV + hv) * 2 + 0] = gred[0] + gred[2];
        a.gate_partials[((int64_t)c * a.HV + hv) * 2 + 1] = gred[1] + gred[3];
      }
    }

    // ---- epilogue 5: dk = accumulator + part from the dq/dk kernel (group-accumulated in fp32)
    const bool l2_k = last && a.rstd_k != nullptr;   // fused L2-norm backward: needs <dk, k> of the finished rows
    {
      float r[KB][16];
#pragma unroll
      for (int b = 0; b < KB; ++b) acc_ld32q(TM_BIG, q, hc * (DK / 2) + b * 32, r[b]);
      tc5::tmem_ld_wait();
      float rk_lo = 0.f, rk_hi = 0.f;
#pragma unroll
      for (int b = 0; b < KB; ++b) {
        FragStore fs;
        FragLoad fk;
        if (l2_k) fk.load(Ks, BT, q * 16, hc * (DK / 2) + b * 32, lane);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int n8 = b * 4 + i, col = n8 * 8 + 2 * t;
          float2 p_lo, p_hi;
          if (!GROUPED) {
            p_lo = unpack_bf16(part16[GROUPED ? 0 : n8][0]);
            p_hi = unpack_bf16(part16[GROUPED ? 0 : n8][1]);
          } else {
            p_lo = part32[GROUPED ? n8 : 0][0];
            p_hi = part32[GROUPED ? n8 : 0][1];
          }
          const float d0 = r[b][4 * i] + p_lo.x, d1 = r[b][4 * i + 1] + p_lo.y;
          const float d2 = r[b][4 * i + 2] + p_hi.x, d3 = r[b][4 * i + 3] + p_hi.y;
          if (!last) {
            if (r_lo < cm.len) *reinterpret_cast<float2*>(dkbuf + r_lo * dkstride + col) = make_float2(d0, d1);
            if (r_hi < cm.len) *reinterpret_cast<float2*>(dkbuf + r_hi * dkstride + col) = make_float2(d2, d3);
          } else {
            fs.set(i, d0, d1, d2, d3);
            if (l2_k) {
              const float2 ka = fk.lo2(i), kb = fk.hi2(i);
              rk_lo += d0 * ka.x + d1 * ka.y;
              rk_hi += d2 * kb.x + d3 * kb.y;
            }
          }
        }
        if (last && !l2_k) fs.store(dWs, BT, q * 16, hc * (DK / 2) + b * 32, lane);
      }
      if (l2_k) {   // r_mk (row sums of M . KK) was consumed before phase 5 ended: its place takes the row dots
        rk_lo = sum_over_t(rk_lo);
        rk_hi = sum_over_t(rk_hi);
        if (t == 0) {
          r_mk[hc * BT + r_lo] = rk_lo;
          r_mk[hc * BT + r_hi] = rk_hi;
        }
      }
    }
    tc5::fence_async_smem();
    tc5::fence_before_sync();
    __syncthreads();
    if (l2_k) {
      // k as passed is the L2-normalised tensor: dk w.r.t. the un-normalised one is (dk - k <dk,k>) rstd.  Both column
      // halves of the dots are there now; every warp forms its block again from the fp32 accumulator (still in
      // tensor memory) and the part it holds in registers, so that the result is rounded once
      const float dot_lo = r_mk[r_lo] + r_mk[BT + r_lo], dot_hi = r_mk[r_hi] + r_mk[BT + r_hi];
      const float rs_lo = r_lo < cm.len ? a.rstd_k[(row0 + r_lo) * a.H + hq] : 0.f;
      const float rs_hi = r_hi < cm.len ? a.rstd_k[(row0 + r_hi) * a.H + hq] : 0.f;
      float r[KB][16];
#pragma unroll
      for (int b = 0; b < KB; ++b) acc_ld32q(TM_BIG, q, hc * (DK / 2) + b * 32, r[b]);
      tc5::tmem_ld_wait();
#pragma unroll
      for (int b = 0; b < KB; ++b) {
        FragLoad fk;
        fk.load(Ks, BT, q * 16, hc * (DK / 2) + b * 32, lane);
        FragStore fs;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int n8 = b * 4 + i;
          float2 p_lo, p_hi;
          if (!GROUPED) {
            p_lo = unpack_bf16(part16[GROUPED ? 0 : n8][0]);
            p_hi = unpack_bf16(part16[GROUPED ? 0 : n8][1]);
          } else {
            p_lo = part32[GROUPED ? n8 : 0][0];
            p_hi = part32[GROUPED ? n8 : 0][1];
          }
          const float2 ka = fk.lo2(i), kb = fk.hi2(i);
          fs.set(i, (r[b][4 * i] + p_lo.x - ka.x * dot_lo) * rs_lo, (r[b][4 * i + 1] + p_lo.y - ka.y * dot_lo) * rs_lo,
                 (r[b][4 * i + 2] + p_hi.x - kb.x * dot_hi) * rs_hi, (r[b][4 * i + 3] + p_hi.y - kb.y * dot_hi) * rs_hi);
        }
        fs.store(dWs, BT, q * 16, hc * (DK / 2) + b * 32, lane);
      }
      tc5::fence_async_smem();
      __syncthreads();
    }
    if (last) {
      if (cm.len == BT) {
        if (tid == 32) {
          tma::store_3d(&maps.dk, (int)cm.row, (hq * DK) / 64, dWs);
          tma::store_commit();
        }
      } else {
        store_tile_swz<BT, DK, NTHREADS>(reinterpret_cast<__nv_bfloat16*>(a.dk) + (row0 * a.H + hq) * DK, (int64_t)a.H * DK, dWs,
                                         cm.len, tid);
      }
    }
  }

  if (tid == 32) tma::store_wait_all<0>();
  if (failed && tid == 0) atomicExch(&g_wy_timeout, 1);
  tc5::fence_before_sync();
  __syncthreads();
  if (warp == 1) tc5::tmem_dealloc(tm, 256);
}

// dA_log[hv] = sum over chunks of the per-chunk partials, same for ddt_bias.  One CTA per head: thread i adds chunks
// i, i + 256, ..., then the 256 sums are added pairwise in a fixed tree (reproducible, no atomics).
__global__ void __launch_bounds__(256) gate_param_reduce_kernel(const b200gdn_chunk_args a) {
  __shared__ float2 part[256];
  const int hv = blockIdx.x, tid = threadIdx.x;
  float sA = 0.f, sB = 0.f;
  for (int c = tid; c < a.n_chunks; c += 256) {
    sA += a.gate_partials[((int64_t)c * a.HV + hv) * 2 + 0];
    sB += a.gate_partials[((int64_t)c * a.HV + hv) * 2 + 1];
  }
  part[tid] = make_float2(sA, sB);
  __syncthreads();
  for (int o = 128; o > 0; o >>= 1) {
    if (tid < o) {
      part[tid].x += part[tid + o].x;
      part[tid].y += part[tid + o].y;
    }
    __syncthreads();
  }
  if (tid == 0) {
    a.dA_log[hv] = part[0].x;
    if (a.ddt_bias) a.ddt_bias[hv] = part[0].y;
  }
}

template <int DK, int DV, bool GROUPED>
int launch(const b200gdn_chunk_args& a, cudaStream_t st) {
  using S = WyTcSmem<DK, DV>;
  if (int e = ensure_smem(bwd_wy_kernel<DK, DV, GROUPED>, S::bytes)) return e;
  WyMaps m;
  const uint64_t pk = (uint64_t)a.H * DK, pv = (uint64_t)a.HV * DV;
  int rc = 0;
  rc |= tma::encode_bf16_panels(&m.k, a.k, a.rows, pk, pk, BT, DK / 64);
  rc |= tma::encode_bf16_panels(&m.v, a.v, a.rows, pv, pv, BT, DV / 64);
  rc |= tma::encode_bf16_panels(&m.du, a.dv2, a.rows, pv, pv, BT, DV / 64);
  rc |= tma::encode_bf16_2d(&m.a, a.A, a.rows, (uint64_t)a.HV * BT, (uint64_t)a.HV * BT, BT);
  rc |= tma::encode_bf16_panels(&m.dv, a.dv, a.rows, pv, pv, BT, DV / 64);
  rc |= tma::encode_bf16_panels(&m.dk, a.dk, a.rows, pk, pk, BT, DK / 64);
  rc |= tma::encode_bf16_panels(&m.h, a.h, (uint64_t)a.n_chunks * a.HV * DK, DV, DV, DK, DV / 64);
  if (rc != 0) return set_error(B200GDN_ERR_CUDA, "bwd_wy: cuTensorMapEncodeTiled failed (%d)", rc);
  dim3 grid(a.n_chunks, a.H);
  bwd_wy_kernel<DK, DV, GROUPED><<<grid, NTHREADS, S::bytes, st>>>(a, m);
  if (int e = check_launch("bwd_wy")) return e;
  if (a.options & B200GDN_PREP_GATE) {
    gate_param_reduce_kernel<<<a.HV, 256, 0, st>>>(a);
    return check_launch("gate_param_reduce");
  }
  return 0;
}

}  // namespace

int launch_bwd_wy(const b200gdn_chunk_args& a, cudaStream_t st) {
  if ((a.options & B200GDN_PREP_GATE) && (a.g == nullptr || a.A_log == nullptr || a.gate_partials == nullptr || a.dA_log == nullptr))
    return set_error(B200GDN_ERR_BAD_ARGUMENT, "bwd_wy: the fused gate needs g (raw), A_log, gate_partials and dA_log");
  if (a.HV > a.H && a.dk_part == nullptr) return set_error(B200GDN_ERR_BAD_ARGUMENT, "bwd_wy: dk_part is required when HV > H");
  const bool grouped = a.HV > a.H;
  if (a.K == 128 && a.V == 128) return grouped ? launch<128, 128, true>(a, st) : launch<128, 128, false>(a, st);
  if (a.K == 64 && a.V == 64) return grouped ? launch<64, 64, true>(a, st) : launch<64, 64, false>(a, st);
  return set_error(B200GDN_ERR_UNSUPPORTED, "bwd_wy: K=%d V=%d not built (64/64 and 128/128 are)", a.K, a.V);
}

// Reads and clears the flag a bounded device wait raises when it expires (synchronises with the device).
int bwd_wy_timeout_flag() {
  int v = 0, zero = 0;
  cudaMemcpyFromSymbol(&v, g_wy_timeout, sizeof(int));
  if (v) cudaMemcpyToSymbol(g_wy_timeout, &zero, sizeof(int));
  return v;
}

}  // namespace gdn
