// Intra-chunk part of the value gradient:
//     dv_local[j] = sum_{i >= j} scale <k_j, q_i> 2^(gamma_i - gamma_j) do_i
// Replaces chunk_bwd_kernel_dv_local (fla/ops/common/chunk_o.py:465-540).  One CTA (4 warps) per (chunk,
// value head) on tcgen05 tensor cores: TMA brings Q, K, do and gamma; P = Q K^T in TMEM; the masked, gated
// and scaled P goes to shared memory as bf16 and is used transposed (MN-major) for dv = P^T do; the result
// leaves through one TMA store into the dv2 buffer, which the reverse scan then completes in place.
#include "tc5_tile.cuh"
#include "tma.cuh"

namespace gdn {
namespace {

constexpr int NTHREADS = 128;
__device__ int g_dvl_timeout = 0;

template <int DK, int DV>
struct DvSmem {
  static constexpr size_t o_q = 0;                       // Q; once P = Q K^T is done, the bf16 P operand
  static constexpr size_t o_k = o_q + (BT * DK * 2 > BT * 128 ? BT * DK * 2 : BT * 128);   // K; later the output staging
  static constexpr size_t o_d = o_k + (BT * DK * 2 > BT * DV * 2 ? BT * DK * 2 : BT * DV * 2);
  static constexpr size_t o_vec = o_d + BT * DV * 2;
  static constexpr size_t bytes = o_vec + BT * 4 + 64 + 1024;
};

struct DvMaps {
  CUtensorMap q, k, d_o, dv2;
};

template <int DK, int DV>
__global__ void __launch_bounds__(NTHREADS, 4) dv_local_kernel(const b200gdn_chunk_args a, const __grid_constant__ DvMaps maps,
                                                            const int pf_dist) {
  using S = DvSmem<DK, DV>;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* Qs = smem + S::o_q;
  unsigned char* Ks = smem + S::o_k;
  unsigned char* Ds = smem + S::o_d;
  unsigned char* Ps = Qs;    // Q is dead once phase 1 has completed
  unsigned char* Stg = Ks;   // and so is K
  float* gs = reinterpret_cast<float*>(smem + S::o_vec);
  uint64_t* bar_ld = reinterpret_cast<uint64_t*>(gs + BT);
  uint64_t* bar_mma = bar_ld + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_mma + 1);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int c = blockIdx.x, hv = blockIdx.y;
  const int G = a.HV / a.H, hq = hv / G;
  const ChunkMeta cm = load_chunk_meta(a.chunk_meta, c);
  const int r_lo = warp * 16 + g, r_hi = r_lo + 8;

  if (tid == 0) {
    tc5::mbar_init(bar_ld, 1);
    tc5::mbar_init(bar_mma, 1);
    tc5::fence_mbar_init();
    // the tiles are on their way while the CTA sets itself up
    tc5::mbar_expect_tx(bar_ld, (uint32_t)(2 * BT * DK * 2 + BT * DV * 2 + BT * 4));
    tma::load_3d(Qs, &maps.q, cm.row, (hq * DK) / 64, bar_ld);
    tma::load_3d(Ks, &maps.k, cm.row, (hq * DK) / 64, bar_ld);
    tma::load_3d(Ds, &maps.d_o, cm.row, (hv * DV) / 64, bar_ld);
    tma::load_1d(gs, gamma_ptr(a.gamma, c, a.HV, hv), BT * 4, bar_ld);
  }
  if (warp == 1) tc5::tmem_alloc(tmem_slot, 128);
  tc5::fence_before_sync();
  __syncthreads();
  tc5::fence_after_sync();
  const uint32_t tm = *tmem_slot;
  const uint32_t TM_P = tm, TM_D = tm;   // P has left tensor memory before dv is accumulated
  PhaseBarrier ph{bar_mma, 0u, &g_dvl_timeout};
  bool failed = false;

  if (tid == 32) {   // while everybody waits for the tiles
    int c2, h2;
    if (successor_cta(pf_dist, c2, h2)) {   // L2 look-ahead for the CTA that will follow this one
      const int row2 = load_chunk_meta(a.chunk_meta, c2).row, hq2 = h2 / G;
      tma::prefetch_3d(&maps.q, row2, (hq2 * DK) / 64);
      tma::prefetch_3d(&maps.k, row2, (hq2 * DK) / 64);
      tma::prefetch_3d(&maps.d_o, row2, (h2 * DV) / 64);
      tma::prefetch_line(gamma_ptr(a.gamma, c2, a.HV, h2));
      tma::prefetch_line(gamma_ptr(a.gamma, c2, a.HV, h2) + 32);
    }
  }
  if (!tc5::mbar_wait(bar_ld, 0)) failed = true;

  if (tid == 0 && !failed) {
    tc5::fence_after_sync();
    issue_mma_t<DK / 16>(TM_P, Operand{tc5::smem_addr(Qs), BT, 0}, Operand{tc5::smem_addr(Ks), BT, 0}, 64, 64, 0);
    ph.commit();
  }
  const float g_lo = gs[r_lo], g_hi = gs[r_hi];
  if (__syncthreads_or(failed || !ph.wait())) {
    failed = true;
  } else {
    // P[i][j] = scale (q_i . k_j) 2^(gamma_i - gamma_j) for j <= i < len (rows past a ragged chunk's end hold
    // another sequence's data and must not leak into the columns of valid rows)
    {
      float r[2][16];
      acc_ld32(TM_P, warp, 0, r[0]);
      acc_ld32(TM_P, warp, 32, r[1]);
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
            v[e] = (ii >= jj && ii < cm.len) ? r[b][4 * i + e] * a.scale * fast_exp2(((e & 2) ? g_hi : g_lo) - gs[jj]) : 0.f;
          }
          fs.set(i, v[0], v[1], v[2], v[3]);
        }
        fs.store(Ps, BT, warp * 16, b * 32, lane);
      }
    }
    tc5::fence_async_smem();
    tc5::fence_before_sync();
    __syncthreads();
    // dv_local = P^T do
    if (tid == 0) {
      tc5::fence_after_sync();
      issue_mma_t<BT / 16>(TM_D, Operand{tc5::smem_addr(Ps), BT, 1}, Operand{tc5::smem_addr(Ds), BT, 1}, 64, DV, 0);
      ph.commit();
    }
    if (__syncthreads_or(!ph.wait())) {
      failed = true;
    } else {
      float r[DV / 32][16];
#pragma unroll
      for (int b = 0; b < DV / 32; ++b) acc_ld32(TM_D, warp, b * 32, r[b]);
      tc5::tmem_ld_wait();
#pragma unroll
      for (int b = 0; b < DV / 32; ++b) {
        FragStore fs;
#pragma unroll
        for (int i = 0; i < 4; ++i) fs.set(i, r[b][4 * i], r[b][4 * i + 1], r[b][4 * i + 2], r[b][4 * i + 3]);
        fs.store(Stg, BT, warp * 16, b * 32, lane);
      }
      tc5::fence_async_smem();
      tc5::fence_before_sync();
      __syncthreads();
      if (cm.len == BT) {
        if (tid == 0) {
          tma::store_3d(&maps.dv2, cm.row, (hv * DV) / 64, Stg);
          tma::store_commit();
          tma::store_wait_all<0>();
        }
      } else {
        store_tile_swz<BT, DV, NTHREADS>(reinterpret_cast<__nv_bfloat16*>(a.dv2) + ((int64_t)cm.row * a.HV + hv) * DV,
                                         (int64_t)a.HV * DV, Stg, cm.len, tid);
      }
    }
  }
  if (failed && tid == 0) atomicExch(&g_dvl_timeout, 1);
  tc5::fence_before_sync();
  __syncthreads();
  if (warp == 1) tc5::tmem_dealloc(tm, 128);
}

template <int DK, int DV>
int launch(const b200gdn_chunk_args& a, cudaStream_t st) {
  using S = DvSmem<DK, DV>;
  if (int e = ensure_smem(dv_local_kernel<DK, DV>, S::bytes)) return e;
  DvMaps m;
  const uint64_t pk = (uint64_t)a.H * DK, pv = (uint64_t)a.HV * DV;
  int rc = 0;
  rc |= tma::encode_bf16_panels(&m.q, a.q, a.rows, pk, pk, BT, DK / 64);
  rc |= tma::encode_bf16_panels(&m.k, a.k, a.rows, pk, pk, BT, DK / 64);
  rc |= tma::encode_bf16_panels(&m.d_o, a.d_o, a.rows, pv, pv, BT, DV / 64);
  rc |= tma::encode_bf16_panels(&m.dv2, a.dv2, a.rows, pv, pv, BT, DV / 64);
  if (rc != 0) return set_error(B200GDN_ERR_CUDA, "dv_local: cuTensorMapEncodeTiled failed (%d)", rc);
  dim3 grid(a.n_chunks, a.HV);
  dv_local_kernel<DK, DV><<<grid, NTHREADS, S::bytes, st>>>(a, m, resident_ctas(dv_local_kernel<DK, DV>, NTHREADS, S::bytes));
  return check_launch("dv_local");
}

}  // namespace

int launch_dv_local(const b200gdn_chunk_args& a, cudaStream_t st) {
  if (a.K == 128 && a.V == 128) return launch<128, 128>(a, st);
  if (a.K == 64 && a.V == 64) return launch<64, 64>(a, st);
  return set_error(B200GDN_ERR_UNSUPPORTED, "dv_local: K=%d V=%d not built (64/64 and 128/128 are)", a.K, a.V);
}

// Reads and clears the flag a bounded device wait raises when it expires (synchronises with the device).
int dv_local_timeout_flag() {
  int v = 0, zero = 0;
  cudaMemcpyFromSymbol(&v, g_dvl_timeout, sizeof(int));
  if (v) cudaMemcpyToSymbol(g_dvl_timeout, &zero, sizeof(int));
  return v;
}

}  // namespace gdn
