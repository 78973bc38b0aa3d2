// Backward of the intra-chunk WY representation (W = A K beta 2^gamma, U = A V beta, A = (I + L)^-1),
// the group sum of dk, and the reverse chunk-local cumsum that turns dG into dg:
//     dKbg = A^T dw,  dVb = A^T du,  dA = strict_tril(dw (K beta 2^gamma)^T + du (V beta)^T)
//     M    = -strict_tril(A^T dA A^T) 2^(gamma_i - gamma_j)
//     dk   = dk_part + dKbg beta 2^gamma + (M K) beta + (M beta_row)^T K
//     dv   = dVb beta
//     dbeta= rowsum(dKbg K) 2^gamma + rowsum(dVb V) + rowsum((M K) K)
//     dG   = dG_part + rowsum(dKbg K) beta 2^gamma + beta rowsum((M K) K) - rowsum(((M beta_row)^T K) K)
// Replaces prepare_wy_repr_bwd_kernel (fla/ops/gated_delta_rule/wy_fast.py:123-251), the sums
// dk + dk2, dg + dg2 and the reverse chunk_local_cumsum (fla/ops/gated_delta_rule/chunk.py:244-246).
// The column scalings of dA and the row scaling of M are applied to accumulators, so K, V, dw, du
// tiles are used as loaded and K K^T is never recomputed.
#include "gdn_common.cuh"

namespace gdn {
namespace {

constexpr int NTHREADS = 128;

template <int DK, int DV>
struct WySmem {
  static constexpr int LDK = DK + PAD, LDV = DV + PAD, LDA = BT + PAD;
  static constexpr int LDS = LDK > LDV ? LDK : LDV;
  static constexpr size_t k_off = 0;
  static constexpr size_t v_off = k_off + sizeof(__nv_bfloat16) * BT * LDK;
  static constexpr size_t dw_off = v_off + sizeof(__nv_bfloat16) * BT * LDV;
  static constexpr size_t du_off = dw_off + sizeof(__nv_bfloat16) * BT * LDK;
  static constexpr size_t a_off = du_off + sizeof(__nv_bfloat16) * BT * LDV;
  static constexpr size_t m_off = a_off + sizeof(__nv_bfloat16) * BT * LDA;
  static constexpr size_t y_off = m_off + sizeof(__nv_bfloat16) * BT * LDA;
  static constexpr size_t stg_off = y_off + sizeof(__nv_bfloat16) * BT * LDA;
  static constexpr size_t vec_off = stg_off + sizeof(__nv_bfloat16) * BT * LDS;
  static constexpr size_t bytes = vec_off + sizeof(float) * 6 * BT;
};

template <int DK, int DV>
__global__ void __launch_bounds__(NTHREADS) wy_bwd_kernel(const b200gdn_chunk_args a) {
  using S = WySmem<DK, DV>;
  extern __shared__ __align__(16) unsigned char smem[];
  __nv_bfloat16* Ks = reinterpret_cast<__nv_bfloat16*>(smem + S::k_off);
  __nv_bfloat16* Vs = reinterpret_cast<__nv_bfloat16*>(smem + S::v_off);
  __nv_bfloat16* dWs = reinterpret_cast<__nv_bfloat16*>(smem + S::dw_off);
  __nv_bfloat16* dUs = reinterpret_cast<__nv_bfloat16*>(smem + S::du_off);
  __nv_bfloat16* As = reinterpret_cast<__nv_bfloat16*>(smem + S::a_off);
  __nv_bfloat16* Ms = reinterpret_cast<__nv_bfloat16*>(smem + S::m_off);
  __nv_bfloat16* Ys = reinterpret_cast<__nv_bfloat16*>(smem + S::y_off);
  __nv_bfloat16* Stg = reinterpret_cast<__nv_bfloat16*>(smem + S::stg_off);
  float* gs = reinterpret_cast<float*>(smem + S::vec_off);
  float* bet = gs + BT;
  float* bge = bet + BT;   // beta 2^gamma
  float* eg = bge + BT;    // 2^gamma
  float* dGs = eg + BT;
  float* dGin = dGs + BT;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int c = blockIdx.x, hq = blockIdx.y;
  const int G = a.HV / a.H;
  const ChunkMeta cm = load_chunk_meta(a.chunk_meta, c);
  const int64_t row0 = cm.row;
  const int r_lo = warp * 16 + g, r_hi = r_lo + 8;

  load_tile_async<DK, NTHREADS>(Ks, reinterpret_cast<const __nv_bfloat16*>(a.k) + (row0 * a.H + hq) * DK,
                                (int64_t)a.H * DK, cm.len, tid);
  cp_async_commit();

  for (int gi = 0; gi < G; ++gi) {
    const int hv = hq * G + gi;
    const bool last = gi == G - 1;
    __syncthreads();
    load_tile_async<DV, NTHREADS>(Vs, reinterpret_cast<const __nv_bfloat16*>(a.v) + (row0 * a.HV + hv) * DV,
                                  (int64_t)a.HV * DV, cm.len, tid);
    load_tile_async<DK, NTHREADS>(dWs, reinterpret_cast<const __nv_bfloat16*>(a.dw) + (row0 * a.HV + hv) * DK,
                                  (int64_t)a.HV * DK, cm.len, tid);
    load_tile_async<DV, NTHREADS>(dUs, reinterpret_cast<const __nv_bfloat16*>(a.dv2) + (row0 * a.HV + hv) * DV,
                                  (int64_t)a.HV * DV, cm.len, tid);
    load_tile_async<BT, NTHREADS>(As, reinterpret_cast<const __nv_bfloat16*>(a.A) + (row0 * a.HV + hv) * BT,
                                  (int64_t)a.HV * BT, cm.len, tid);
    cp_async_commit();
    load_gamma(gs, a.gamma, cm.row, cm.len, a.HV, hv, tid);
    if (tid < BT) {
      bool ok = tid < cm.len;
      bet[tid] = ok ? a.beta[(row0 + tid) * a.HV + hv] : 0.f;
      dGin[tid] = ok ? a.dG[(row0 + tid) * a.HV + hv] : 0.f;
    }
    cp_async_wait<0>();
    __syncthreads();
    if (tid < BT) {
      float e = exp2f(gs[tid]);
      eg[tid] = e;
      bge[tid] = bet[tid] * e;
    }
    __syncthreads();

    const float g_lo = gs[r_lo], g_hi = gs[r_hi];
    const float b_lo = bet[r_lo], b_hi = bet[r_hi];
    const float bg_lo = bge[r_lo], bg_hi = bge[r_hi];

    // dA (strictly lower) as A fragments
    uint32_t dafrag[4][4];
    {
      float acc1[8][4], acc2[8][4];
      zero_acc<8>(acc1);
      zero_acc<8>(acc2);
      warp_mma<8, DK / 16, AMajor::Row, BMajor::NK>(acc1, dWs + warp * 16 * S::LDK, S::LDK, Ks, S::LDK, lane);
      warp_mma<8, DV / 16, AMajor::Row, BMajor::NK>(acc2, dUs + warp * 16 * S::LDV, S::LDV, Vs, S::LDV, lane);
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          int i = (e & 2) ? r_hi : r_lo;
          int j = nt * 8 + 2 * t + (e & 1);
          acc1[nt][e] = (i > j) ? acc1[nt][e] * bge[j] + acc2[nt][e] * bet[j] : 0.f;
        }
      }
      acc_to_afrag<8>(dafrag, acc1);
    }
    // Y = dA A^T
    {
      float acc[8][4];
      zero_acc<8>(acc);
      warp_mma_ra<8, 4, BMajor::NK>(acc, dafrag, As, S::LDA, lane);
      acc_to_smem<8>(Ys + warp * 16 * S::LDA, S::LDA, acc, lane);
    }
    __syncthreads();
    // X = A^T Y ; M = -strict_tril(X) 2^(gamma_i - gamma_j)
    uint32_t mfrag[4][4];
    {
      float acc[8][4];
      zero_acc<8>(acc);
      warp_mma<8, BT / 16, AMajor::Trans, BMajor::KN>(acc, As + warp * 16, S::LDA, Ys, S::LDA, lane);
      float m2[8][4];
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          int i = (e & 2) ? r_hi : r_lo;
          int j = nt * 8 + 2 * t + (e & 1);
          float gi_ = (e & 2) ? g_hi : g_lo;
          float m = (i > j) ? -acc[nt][e] * exp2f(gi_ - gs[j]) : 0.f;
          acc[nt][e] = m;
          m2[nt][e] = m * ((e & 2) ? b_hi : b_lo);
        }
      }
      acc_to_afrag<8>(mfrag, acc);
      acc_to_smem<8>(Ms + warp * 16 * S::LDA, S::LDA, m2, lane);
    }

    float dk[DK / 8][4];
    float r_kbg_lo, r_kbg_hi, r_mk_lo, r_mk_hi, r_m2_lo, r_m2_hi, r_vb_lo, r_vb_hi;
    {
      float tmp[DK / 8][4];
      zero_acc<DK / 8>(tmp);
      warp_mma<DK / 8, BT / 16, AMajor::Trans, BMajor::KN>(tmp, As + warp * 16, S::LDA, dWs, S::LDK, lane);
      row_dot<DK / 8>(r_kbg_lo, r_kbg_hi, tmp, Ks + warp * 16 * S::LDK, S::LDK, lane);
#pragma unroll
      for (int nt = 0; nt < DK / 8; ++nt) {
        dk[nt][0] = tmp[nt][0] * bg_lo; dk[nt][1] = tmp[nt][1] * bg_lo;
        dk[nt][2] = tmp[nt][2] * bg_hi; dk[nt][3] = tmp[nt][3] * bg_hi;
      }
      zero_acc<DK / 8>(tmp);
      warp_mma_ra<DK / 8, 4, BMajor::KN>(tmp, mfrag, Ks, S::LDK, lane);
      row_dot<DK / 8>(r_mk_lo, r_mk_hi, tmp, Ks + warp * 16 * S::LDK, S::LDK, lane);
#pragma unroll
      for (int nt = 0; nt < DK / 8; ++nt) {
        dk[nt][0] += tmp[nt][0] * b_lo; dk[nt][1] += tmp[nt][1] * b_lo;
        dk[nt][2] += tmp[nt][2] * b_hi; dk[nt][3] += tmp[nt][3] * b_hi;
      }
      __syncthreads();  // Ms complete
      zero_acc<DK / 8>(tmp);
      warp_mma<DK / 8, BT / 16, AMajor::Trans, BMajor::KN>(tmp, Ms + warp * 16, S::LDA, Ks, S::LDK, lane);
      row_dot<DK / 8>(r_m2_lo, r_m2_hi, tmp, Ks + warp * 16 * S::LDK, S::LDK, lane);
#pragma unroll
      for (int nt = 0; nt < DK / 8; ++nt) {
        dk[nt][0] += tmp[nt][0]; dk[nt][1] += tmp[nt][1]; dk[nt][2] += tmp[nt][2]; dk[nt][3] += tmp[nt][3];
      }
    }
    // group accumulation of dk in the fp32 buffer that already holds the dqkwg part
    {
      float* buf = a.dk_part + (row0 * a.H + hq) * DK;
      const int64_t stride = (int64_t)a.H * DK;
#pragma unroll
      for (int nt = 0; nt < DK / 8; ++nt) {
        const int col = nt * 8 + 2 * t;
        if (r_lo < cm.len) {
          float2* p = reinterpret_cast<float2*>(buf + r_lo * stride + col);
          float2 o = *p;
          dk[nt][0] += o.x; dk[nt][1] += o.y;
          if (!last) *p = make_float2(dk[nt][0], dk[nt][1]);
        }
        if (r_hi < cm.len) {
          float2* p = reinterpret_cast<float2*>(buf + r_hi * stride + col);
          float2 o = *p;
          dk[nt][2] += o.x; dk[nt][3] += o.y;
          if (!last) *p = make_float2(dk[nt][2], dk[nt][3]);
        }
      }
    }
    if (last) {
      acc_to_smem<DK / 8>(Stg + warp * 16 * S::LDS, S::LDS, dk, lane);
    }
    __syncthreads();
    if (last) {
      // staging row stride is LDS; store_tile assumes COLS + PAD, which equals LDS when DK >= DV
      store_tile<BT, DK, NTHREADS>(reinterpret_cast<__nv_bfloat16*>(a.dk) + (row0 * a.H + hq) * DK, (int64_t)a.H * DK, Stg,
                                   cm.len, tid);
    }
    __syncthreads();

    // dv = (A^T du) beta
    {
      float tmp[DV / 8][4];
      zero_acc<DV / 8>(tmp);
      warp_mma<DV / 8, BT / 16, AMajor::Trans, BMajor::KN>(tmp, As + warp * 16, S::LDA, dUs, S::LDV, lane);
      row_dot<DV / 8>(r_vb_lo, r_vb_hi, tmp, Vs + warp * 16 * S::LDV, S::LDV, lane);
#pragma unroll
      for (int nt = 0; nt < DV / 8; ++nt) {
        tmp[nt][0] *= b_lo; tmp[nt][1] *= b_lo; tmp[nt][2] *= b_hi; tmp[nt][3] *= b_hi;
      }
      acc_to_smem<DV / 8>(Stg + warp * 16 * S::LDV, S::LDV, tmp, lane);
    }
    if (t == 0) {
      float db_lo = r_kbg_lo * eg[r_lo] + r_vb_lo + r_mk_lo;
      float db_hi = r_kbg_hi * eg[r_hi] + r_vb_hi + r_mk_hi;
      if (r_lo < cm.len) a.dbeta[(row0 + r_lo) * a.HV + hv] = db_lo;
      if (r_hi < cm.len) a.dbeta[(row0 + r_hi) * a.HV + hv] = db_hi;
      dGs[r_lo] = r_kbg_lo * bg_lo + b_lo * r_mk_lo - r_m2_lo + dGin[r_lo];
      dGs[r_hi] = r_kbg_hi * bg_hi + b_hi * r_mk_hi - r_m2_hi + dGin[r_hi];
    }
    __syncthreads();
    store_tile<BT, DV, NTHREADS>(reinterpret_cast<__nv_bfloat16*>(a.dv) + (row0 * a.HV + hv) * DV, (int64_t)a.HV * DV, Stg,
                                 cm.len, tid);
    if (tid < cm.len) {
      float s = 0.f;
      for (int j = BT - 1; j >= tid; --j) s += dGs[j];
      a.dg[(row0 + tid) * a.HV + hv] = s;
    }
  }
}

template <int DK, int DV>
int launch(const b200gdn_chunk_args& a, cudaStream_t st) {
  using S = WySmem<DK, DV>;
  static_assert(DK == DV, "staging stride assumes equal head dimensions");
  if (int e = ensure_smem(wy_bwd_kernel<DK, DV>, S::bytes)) return e;
  dim3 grid(a.n_chunks, a.H);
  wy_bwd_kernel<DK, DV><<<grid, NTHREADS, S::bytes, st>>>(a);
  return check_launch("wy_bwd");
}

}  // namespace

int launch_wy_bwd(const b200gdn_chunk_args& a, cudaStream_t st) {
  if (a.K == 128 && a.V == 128) return launch<128, 128>(a, st);
  if (a.K == 64 && a.V == 64) return launch<64, 64>(a, st);
  return set_error(B200GDN_ERR_UNSUPPORTED, "wy_bwd: K=%d V=%d not built (64/64 and 128/128 are)", a.K, a.V);
}

}  // namespace gdn
