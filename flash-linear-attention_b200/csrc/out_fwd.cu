// Chunk output:  o = scale [ (Q h_c) 2^gamma + tril(Q K^T 2^(gamma_i - gamma_j)) v_new ].
// Replaces chunk_fwd_kernel_o (fla/ops/common/chunk_o.py:56-153).  One CTA (4 warps) per (chunk, value
// head), tcgen05 tensor cores with a 128-column TMEM accumulator used for one product after the other:
//   load    : one thread issues the TMA copies (Q, K, the 128 x 128 state snapshot, gamma) before the CTA has
//             even set itself up, and pulls the tiles of the CTA that will follow this one into L2;
//   phase 1a: P = Q K^T;      epilogue: P masked and gated -> bf16 operand tile; K is dead, v_new is loaded over it;
//   phase 1b: O = Q h;        epilogue: O rows scaled by 2^gamma_i in place (tcgen05.ld / tcgen05.st);
//   phase 2 : O += P v_new;   epilogue: scale, bf16, one TMA store (plain predicated stores for a ragged chunk).
// 128 TMEM columns and ~73 KiB of shared memory per CTA: three CTAs per SM hide each other's latencies.
#include "tc5_tile.cuh"
#include "tma.cuh"

namespace gdn {
namespace {

constexpr int NTHREADS = 128;
__device__ int g_out_timeout = 0;

template <int DK, int DV>
struct OutSmem {
  static constexpr size_t o_q = 0;                       // Q; later the output staging tile
  static constexpr size_t o_k = o_q + (BT * DK * 2 > BT * DV * 2 ? BT * DK * 2 : BT * DV * 2);
  static constexpr size_t o_h = o_k + (BT * DK * 2 > BT * DV * 2 ? BT * DK * 2 : BT * DV * 2);   // K, then v_new
  static constexpr size_t o_p = o_h + DK * DV * 2;
  static constexpr size_t o_vec = o_p + BT * 128;
  static constexpr size_t bytes = o_vec + BT * 4 + 64 + 1024;
};

struct OutMaps {
  CUtensorMap q, k, vn, h, o;
};

template <int DK, int DV>
__global__ void __launch_bounds__(NTHREADS, 3) out_fwd_kernel(const b200gdn_chunk_args a, const __grid_constant__ OutMaps maps,
                                                              const int pf_dist) {
  using S = OutSmem<DK, DV>;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* Qs = smem + S::o_q;
  unsigned char* Ks = smem + S::o_k;
  unsigned char* Vn = smem + S::o_k;   // takes K's place once P = Q K^T is done
  unsigned char* Hs = smem + S::o_h;
  unsigned char* Ps = smem + S::o_p;
  float* gs = reinterpret_cast<float*>(smem + S::o_vec);
  uint64_t* bar_qk = reinterpret_cast<uint64_t*>(gs + BT);
  uint64_t* bar_h = bar_qk + 1;
  uint64_t* bar_v = bar_qk + 2;
  uint64_t* bar_mma = bar_qk + 3;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_qk + 4);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int c = blockIdx.x, hv = blockIdx.y;
  const int G = a.HV / a.H, hq = hv / G;
  const ChunkMeta cm = load_chunk_meta(a.chunk_meta, c);
  const int r_lo = warp * 16 + g, r_hi = r_lo + 8;

  if (tid == 0) {
    tc5::mbar_init(bar_qk, 1);
    tc5::mbar_init(bar_h, 1);
    tc5::mbar_init(bar_v, 1);
    tc5::mbar_init(bar_mma, 1);
    tc5::fence_mbar_init();
    tc5::mbar_expect_tx(bar_qk, (uint32_t)(2 * BT * DK * 2 + BT * 4));
    tma::load_3d(Qs, &maps.q, cm.row, (hq * DK) / 64, bar_qk);
    tma::load_3d(Ks, &maps.k, cm.row, (hq * DK) / 64, bar_qk);
    tma::load_1d(gs, gamma_ptr(a.gamma, c, a.HV, hv), BT * 4, bar_qk);
    tc5::mbar_expect_tx(bar_h, (uint32_t)(DK * DV * 2));
    tma::load_3d(Hs, &maps.h, (c * a.HV + hv) * DK, 0, bar_h);
    tma::prefetch_3d(&maps.vn, cm.row, (hv * DV) / 64);   // loaded late (over K): have it in L2 by then
  }
  if (warp == 1) tc5::tmem_alloc(tmem_slot, 128);
  tc5::fence_before_sync();
  __syncthreads();
  tc5::fence_after_sync();
  const uint32_t tm = *tmem_slot;
  PhaseBarrier ph{bar_mma, 0u, &g_out_timeout};
  bool failed = false;

  if (tid == 32) {   // while everybody waits for the tiles
    int c2, h2;
    if (successor_cta(pf_dist, c2, h2)) {   // L2 look-ahead for the CTA that will follow this one
      const int row2 = load_chunk_meta(a.chunk_meta, c2).row, hq2 = h2 / G;
      tma::prefetch_3d(&maps.q, row2, (hq2 * DK) / 64);
      tma::prefetch_3d(&maps.k, row2, (hq2 * DK) / 64);
      tma::prefetch_3d(&maps.h, (c2 * a.HV + h2) * DK, 0);
      tma::prefetch_line(gamma_ptr(a.gamma, c2, a.HV, h2));
      tma::prefetch_line(gamma_ptr(a.gamma, c2, a.HV, h2) + 32);
    }
  }
  if (!tc5::mbar_wait(bar_qk, 0)) failed = true;

  // ---- phase 1a: P = Q K^T
  if (tid == 0 && !failed) {
    tc5::fence_after_sync();
    issue_mma_t<DK / 16>(tm, Operand{tc5::smem_addr(Qs), BT, 0}, Operand{tc5::smem_addr(Ks), BT, 0}, 64, 64, 0);
    ph.commit();
  }
  const float g_lo = gs[r_lo], g_hi = gs[r_hi];
  if (__syncthreads_or(failed || !ph.wait())) {
    failed = true;
  } else {
    // ---- epilogue 1a: P masked and gated -> bf16 operand tile
    {
      float r[2][16];
      acc_ld32(tm, warp, 0, r[0]);
      acc_ld32(tm, warp, 32, r[1]);
      tc5::tmem_ld_wait();
#pragma unroll
      for (int b = 0; b < 2; ++b) {
        FragStore fs;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int j0 = b * 32 + i * 8 + 2 * t;
          float v[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int ii = (e & 2) ? r_hi : r_lo, jj = j0 + (e & 1);
            v[e] = (ii >= jj) ? r[b][4 * i + e] * fast_exp2(((e & 2) ? g_hi : g_lo) - gs[jj]) : 0.f;
          }
          fs.set(i, v[0], v[1], v[2], v[3]);
        }
        fs.store(Ps, BT, warp * 16, b * 32, lane);
      }
    }
    if (!tc5::mbar_wait(bar_h, 0)) failed = true;
    tc5::fence_async_smem();
    tc5::fence_before_sync();
    if (__syncthreads_or(failed)) {
      failed = true;
    } else {
      // ---- phase 1b: O = Q h (over the columns P has left); v_new arrives over K meanwhile
      if (tid == 0) {
        tc5::fence_after_sync();
        issue_mma_t<DK / 16>(tm, Operand{tc5::smem_addr(Qs), BT, 0}, Operand{tc5::smem_addr(Hs), DK, 1}, 64, DV, 0);
        ph.commit();
        tc5::mbar_expect_tx(bar_v, (uint32_t)(BT * DV * 2));
        tma::load_3d(Vn, &maps.vn, cm.row, (hv * DV) / 64, bar_v);
      }
      if (__syncthreads_or(!ph.wait())) {
        failed = true;
      } else {
        // ---- epilogue 1b: O rows scaled by 2^gamma_i in place
        {
          const float e_lo = fast_exp2(g_lo), e_hi = fast_exp2(g_hi);
          float r[DV / 32][16];
#pragma unroll
          for (int b = 0; b < DV / 32; ++b) acc_ld32(tm, warp, b * 32, r[b]);
          tc5::tmem_ld_wait();
#pragma unroll
          for (int b = 0; b < DV / 32; ++b) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              r[b][4 * i] *= e_lo; r[b][4 * i + 1] *= e_lo; r[b][4 * i + 2] *= e_hi; r[b][4 * i + 3] *= e_hi;
            }
            tc5::tmem_st_16x256b_x4(tm + ((uint32_t)(warp * 32) << 16) + b * 32, r[b]);
          }
          tc5::tmem_st_wait();
        }
        if (!tc5::mbar_wait(bar_v, 0)) failed = true;
        tc5::fence_before_sync();
        if (__syncthreads_or(failed)) {
          failed = true;
        } else {
          // ---- phase 2: O += P v_new
          if (tid == 0) {
            tc5::fence_after_sync();
            issue_mma_t<BT / 16>(tm, Operand{tc5::smem_addr(Ps), BT, 0}, Operand{tc5::smem_addr(Vn), BT, 1}, 64, DV, 1);
            ph.commit();
          }
          if (__syncthreads_or(!ph.wait())) {
            failed = true;
          } else {
            // ---- epilogue 2: scale, bf16 -> staging tile (over Q) -> global
            float r[DV / 32][16];
#pragma unroll
            for (int b = 0; b < DV / 32; ++b) acc_ld32(tm, warp, b * 32, r[b]);
            tc5::tmem_ld_wait();
#pragma unroll
            for (int b = 0; b < DV / 32; ++b) {
              FragStore fs;
#pragma unroll
              for (int i = 0; i < 4; ++i)
                fs.set(i, r[b][4 * i] * a.scale, r[b][4 * i + 1] * a.scale, r[b][4 * i + 2] * a.scale, r[b][4 * i + 3] * a.scale);
              fs.store(Qs, BT, warp * 16, b * 32, lane);
            }
            tc5::fence_async_smem();
            tc5::fence_before_sync();
            __syncthreads();
            if (cm.len == BT) {
              if (tid == 0) {
                tma::store_3d(&maps.o, cm.row, (hv * DV) / 64, Qs);
                tma::store_commit();
                tma::store_wait_all<0>();
              }
            } else {
              store_tile_swz<BT, DV, NTHREADS>(reinterpret_cast<__nv_bfloat16*>(a.o) + ((int64_t)cm.row * a.HV + hv) * DV,
                                               (int64_t)a.HV * DV, Qs, cm.len, tid);
            }
          }
        }
      }
    }
  }
  if (failed && tid == 0) atomicExch(&g_out_timeout, 1);
  tc5::fence_before_sync();
  __syncthreads();
  if (warp == 1) tc5::tmem_dealloc(tm, 128);
}

template <int DK, int DV>
int launch(const b200gdn_chunk_args& a, cudaStream_t st) {
  using S = OutSmem<DK, DV>;
  if (int e = ensure_smem(out_fwd_kernel<DK, DV>, S::bytes)) return e;
  OutMaps m;
  const uint64_t pk = (uint64_t)a.H * DK, pv = (uint64_t)a.HV * DV;
  int rc = 0;
  rc |= tma::encode_bf16_panels(&m.q, a.q, a.rows, pk, pk, BT, DK / 64);
  rc |= tma::encode_bf16_panels(&m.k, a.k, a.rows, pk, pk, BT, DK / 64);
  rc |= tma::encode_bf16_panels(&m.vn, a.v_new, a.rows, pv, pv, BT, DV / 64);
  rc |= tma::encode_bf16_panels(&m.h, a.h, (uint64_t)a.n_chunks * a.HV * DK, DV, DV, DK, DV / 64);
  rc |= tma::encode_bf16_panels(&m.o, a.o, a.rows, pv, pv, BT, DV / 64);
  if (rc != 0) return set_error(B200GDN_ERR_CUDA, "out_fwd: cuTensorMapEncodeTiled failed (%d)", rc);
  dim3 grid(a.n_chunks, a.HV);
  out_fwd_kernel<DK, DV><<<grid, NTHREADS, S::bytes, st>>>(a, m, resident_ctas(out_fwd_kernel<DK, DV>, NTHREADS, S::bytes));
  return check_launch("out_fwd");
}

}  // namespace

int launch_out_fwd(const b200gdn_chunk_args& a, cudaStream_t st) {
  if (a.K == 128 && a.V == 128) return launch<128, 128>(a, st);
  if (a.K == 64 && a.V == 64) return launch<64, 64>(a, st);
  return set_error(B200GDN_ERR_UNSUPPORTED, "out_fwd: K=%d V=%d not built (64/64 and 128/128 are)", a.K, a.V);
}

// Reads and clears the flag a bounded device wait raises when it expires (synchronises with the device).
int out_fwd_timeout_flag() {
  int v = 0, zero = 0;
  cudaMemcpyFromSymbol(&v, g_out_timeout, sizeof(int));
  if (v) cudaMemcpyToSymbol(g_out_timeout, &zero, sizeof(int));
  return v;
}

}  // namespace gdn
