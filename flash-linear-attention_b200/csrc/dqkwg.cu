// Chunk-local gradients of q, k, w and of the cumulative gate:
//     dP   = tril(do v_new^T 2^(gamma_i - gamma_j)) scale
//     dq   = scale (do h^T) 2^gamma + dP k
//     dk   = dP^T q + (v_new dh^T) 2^(gamma_last - gamma)
//     dw   = -dv2 h^T
//     dG_i = <dq_i,q_i> - <dk_i,k_i>  (+ at the last valid row: 2^gamma_last <h,dh> + sum_i <dk_state_i,k_i>)
// Replaces chunk_bwd_kernel_dqkwg (fla/ops/common/chunk_o.py:172-342) and the group sum over value
// heads that follows it (:774-776).  One CTA per (chunk, q/k head) loops over the value heads of its
// group, so dq and dk are reduced over the group deterministically and without atomics.
#include "gdn_common.cuh"

namespace gdn {
namespace {

constexpr int NTHREADS = 128;

template <int DK, int DV>
struct DqkwgSmem {
  static constexpr int LDK = DK + PAD, LDV = DV + PAD, LDP = BT + PAD;
  static constexpr size_t q_off = 0;
  static constexpr size_t k_off = q_off + sizeof(__nv_bfloat16) * BT * LDK;
  static constexpr size_t do_off = k_off + sizeof(__nv_bfloat16) * BT * LDK;
  static constexpr size_t vn_off = do_off + sizeof(__nv_bfloat16) * BT * LDV;
  static constexpr size_t d2_off = vn_off + sizeof(__nv_bfloat16) * BT * LDV;
  static constexpr size_t h_off = d2_off + sizeof(__nv_bfloat16) * BT * LDV;
  static constexpr size_t dh_off = h_off + sizeof(__nv_bfloat16) * DK * LDV;
  static constexpr size_t p_off = dh_off + sizeof(__nv_bfloat16) * DK * LDV;
  static constexpr size_t stg_off = p_off + sizeof(__nv_bfloat16) * BT * LDP;
  static constexpr size_t vec_off = stg_off + sizeof(__nv_bfloat16) * BT * LDK;
  static constexpr size_t bytes = vec_off + sizeof(float) * (2 * BT + 16);
};

// acc (+)= buf ; buf = acc   on the rows a warp owns (fp32 [rows][stride] global, rows < valid)
template <int NT>
__device__ __forceinline__ void rmw_global(float (&acc)[NT][4], float* buf, int64_t stride, int valid, int warp, int lane,
                                           bool add, bool store) {
  const int g = lane >> 2, t = lane & 3;
  const int r_lo = warp * 16 + g, r_hi = r_lo + 8;
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    const int col = nt * 8 + 2 * t;
    if (r_lo < valid) {
      float2* p = reinterpret_cast<float2*>(buf + r_lo * stride + col);
      if (add) { float2 o = *p; acc[nt][0] += o.x; acc[nt][1] += o.y; }
      if (store) *p = make_float2(acc[nt][0], acc[nt][1]);
    }
    if (r_hi < valid) {
      float2* p = reinterpret_cast<float2*>(buf + r_hi * stride + col);
      if (add) { float2 o = *p; acc[nt][2] += o.x; acc[nt][3] += o.y; }
      if (store) *p = make_float2(acc[nt][2], acc[nt][3]);
    }
  }
}

template <int DK, int DV>
__global__ void __launch_bounds__(NTHREADS) dqkwg_kernel(const b200gdn_chunk_args a) {
  using S = DqkwgSmem<DK, DV>;
  extern __shared__ __align__(16) unsigned char smem[];
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem + S::q_off);
  __nv_bfloat16* Ks = reinterpret_cast<__nv_bfloat16*>(smem + S::k_off);
  __nv_bfloat16* Ds = reinterpret_cast<__nv_bfloat16*>(smem + S::do_off);
  __nv_bfloat16* Vn = reinterpret_cast<__nv_bfloat16*>(smem + S::vn_off);
  __nv_bfloat16* D2 = reinterpret_cast<__nv_bfloat16*>(smem + S::d2_off);
  __nv_bfloat16* Hs = reinterpret_cast<__nv_bfloat16*>(smem + S::h_off);
  __nv_bfloat16* dHs = reinterpret_cast<__nv_bfloat16*>(smem + S::dh_off);
  __nv_bfloat16* Ps = reinterpret_cast<__nv_bfloat16*>(smem + S::p_off);
  __nv_bfloat16* Stg = reinterpret_cast<__nv_bfloat16*>(smem + S::stg_off);
  float* gs = reinterpret_cast<float*>(smem + S::vec_off);
  float* dGs = gs + BT;
  float* red = dGs + BT;  // [0..3] <h,dh> partials, [4..7] <dk_state,k> partials

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int c = blockIdx.x, hq = blockIdx.y;
  const int G = a.HV / a.H;
  const ChunkMeta cm = load_chunk_meta(a.chunk_meta, c);
  const int64_t row0 = cm.row;
  const int r_lo = warp * 16 + g, r_hi = r_lo + 8;

  load_tile_async<DK, NTHREADS>(Qs, reinterpret_cast<const __nv_bfloat16*>(a.q) + (row0 * a.H + hq) * DK,
                                (int64_t)a.H * DK, cm.len, tid);
  load_tile_async<DK, NTHREADS>(Ks, reinterpret_cast<const __nv_bfloat16*>(a.k) + (row0 * a.H + hq) * DK,
                                (int64_t)a.H * DK, cm.len, tid);
  cp_async_commit();

  for (int gi = 0; gi < G; ++gi) {
    const int hv = hq * G + gi;
    const bool first = gi == 0, last = gi == G - 1;
    __syncthreads();  // previous head fully consumed
    load_tile_async<DV, NTHREADS>(Ds, reinterpret_cast<const __nv_bfloat16*>(a.d_o) + (row0 * a.HV + hv) * DV,
                                  (int64_t)a.HV * DV, cm.len, tid);
    load_tile_async<DV, NTHREADS>(Vn, reinterpret_cast<const __nv_bfloat16*>(a.v_new) + (row0 * a.HV + hv) * DV,
                                  (int64_t)a.HV * DV, cm.len, tid);
    load_tile_async<DV, NTHREADS>(D2, reinterpret_cast<const __nv_bfloat16*>(a.dv2) + (row0 * a.HV + hv) * DV,
                                  (int64_t)a.HV * DV, cm.len, tid);
    load_rows_async<DK, DV, NTHREADS>(Hs, reinterpret_cast<const __nv_bfloat16*>(a.h) + ((int64_t)c * a.HV + hv) * DK * DV,
                                      DV, tid);
    load_rows_async<DK, DV, NTHREADS>(dHs, reinterpret_cast<const __nv_bfloat16*>(a.dh) + ((int64_t)c * a.HV + hv) * DK * DV,
                                      DV, tid);
    cp_async_commit();
    load_gamma(gs, a.gamma, cm.row, cm.len, a.HV, hv, tid);
    cp_async_wait<0>();
    __syncthreads();

    const float g_lo = gs[r_lo], g_hi = gs[r_hi], glast = gs[BT - 1];

    // <h, dh> partial sums
    {
      float s = 0.f;
      for (int idx = tid; idx < DK * DV / 2; idx += NTHREADS) {
        int r = idx / (DV / 2), col = (idx % (DV / 2)) * 2;
        float2 x = unpack_bf16(*reinterpret_cast<const uint32_t*>(Hs + r * S::LDV + col));
        float2 y = unpack_bf16(*reinterpret_cast<const uint32_t*>(dHs + r * S::LDV + col));
        s += x.x * y.x + x.y * y.y;
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
      if (lane == 0) red[warp] = s;
    }

    // dP
    uint32_t pfrag[4][4];
    {
      float acc[8][4];
      zero_acc<8>(acc);
      warp_mma<8, DV / 16, AMajor::Row, BMajor::NK>(acc, Ds + warp * 16 * S::LDV, S::LDV, Vn, S::LDV, lane);
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          int i = (e & 2) ? r_hi : r_lo;
          int j = nt * 8 + 2 * t + (e & 1);
          float gi_ = (e & 2) ? g_hi : g_lo;
          acc[nt][e] = (i >= j) ? acc[nt][e] * a.scale * exp2f(gi_ - gs[j]) : 0.f;
        }
      }
      acc_to_afrag<8>(pfrag, acc);
      acc_to_smem<8>(Ps + warp * 16 * S::LDP, S::LDP, acc, lane);
    }

    // dq
    float rq_lo, rq_hi;
    {
      float acc[DK / 8][4];
      zero_acc<DK / 8>(acc);
      warp_mma<DK / 8, DV / 16, AMajor::Row, BMajor::NK>(acc, Ds + warp * 16 * S::LDV, S::LDV, Hs, S::LDV, lane);
      const float s_lo = a.scale * exp2f(g_lo), s_hi = a.scale * exp2f(g_hi);
#pragma unroll
      for (int nt = 0; nt < DK / 8; ++nt) {
        acc[nt][0] *= s_lo; acc[nt][1] *= s_lo; acc[nt][2] *= s_hi; acc[nt][3] *= s_hi;
      }
      warp_mma_ra<DK / 8, 4, BMajor::KN>(acc, pfrag, Ks, S::LDK, lane);
      row_dot<DK / 8>(rq_lo, rq_hi, acc, Qs + warp * 16 * S::LDK, S::LDK, lane);
      if (G > 1) {
        float* buf = a.dq_acc + (row0 * a.H + hq) * DK;
        rmw_global<DK / 8>(acc, buf, (int64_t)a.H * DK, cm.len, warp, lane, !first, !last);
      }
      if (last) acc_to_smem<DK / 8>(Stg + warp * 16 * S::LDK, S::LDK, acc, lane);
    }
    __syncthreads();  // Ps and (on the last head) the dq staging tile are complete
    if (last)
      store_tile<BT, DK, NTHREADS>(reinterpret_cast<__nv_bfloat16*>(a.dq) + (row0 * a.H + hq) * DK, (int64_t)a.H * DK, Stg,
                                   cm.len, tid);

    // dk
    float rk_lo, rk_hi, rs_lo, rs_hi;
    {
      float acc[DK / 8][4];
      zero_acc<DK / 8>(acc);
      warp_mma<DK / 8, DV / 16, AMajor::Row, BMajor::NK>(acc, Vn + warp * 16 * S::LDV, S::LDV, dHs, S::LDV, lane);
      const float e_lo = exp2f(glast - g_lo), e_hi = exp2f(glast - g_hi);
#pragma unroll
      for (int nt = 0; nt < DK / 8; ++nt) {
        acc[nt][0] *= e_lo; acc[nt][1] *= e_lo; acc[nt][2] *= e_hi; acc[nt][3] *= e_hi;
      }
      row_dot<DK / 8>(rs_lo, rs_hi, acc, Ks + warp * 16 * S::LDK, S::LDK, lane);
      warp_mma<DK / 8, BT / 16, AMajor::Trans, BMajor::KN>(acc, Ps + warp * 16, S::LDP, Qs, S::LDK, lane);
      row_dot<DK / 8>(rk_lo, rk_hi, acc, Ks + warp * 16 * S::LDK, S::LDK, lane);
      float* buf = a.dk_part + (row0 * a.H + hq) * DK;
      rmw_global<DK / 8>(acc, buf, (int64_t)a.H * DK, cm.len, warp, lane, !first, true);
    }
    // gate gradient rows and the tail partial of this warp
    {
      float sk = (t == 0) ? rs_lo + rs_hi : 0.f;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) sk += __shfl_xor_sync(0xffffffffu, sk, o);
      if (lane == 0) red[4 + warp] = sk;
      if (t == 0) {
        dGs[r_lo] = rq_lo - rk_lo;
        dGs[r_hi] = rq_hi - rk_hi;
      }
    }
    __syncthreads();  // dq store has drained the staging tile; dGs/red are complete

    // dw = -dv2 h^T
    {
      float acc[DK / 8][4];
      zero_acc<DK / 8>(acc);
      warp_mma<DK / 8, DV / 16, AMajor::Row, BMajor::NK, true>(acc, D2 + warp * 16 * S::LDV, S::LDV, Hs, S::LDV, lane);
      acc_to_smem<DK / 8>(Stg + warp * 16 * S::LDK, S::LDK, acc, lane);
    }
    if (tid < cm.len) {
      float tail = exp2f(glast) * (red[0] + red[1] + red[2] + red[3]) + (red[4] + red[5] + red[6] + red[7]);
      a.dG[(row0 + tid) * a.HV + hv] = dGs[tid] + (tid == cm.len - 1 ? tail : 0.f);
    }
    __syncthreads();
    store_tile<BT, DK, NTHREADS>(reinterpret_cast<__nv_bfloat16*>(a.dw) + (row0 * a.HV + hv) * DK, (int64_t)a.HV * DK, Stg,
                                 cm.len, tid);
  }
}

template <int DK, int DV>
int launch(const b200gdn_chunk_args& a, cudaStream_t st) {
  using S = DqkwgSmem<DK, DV>;
  if (int e = ensure_smem(dqkwg_kernel<DK, DV>, S::bytes)) return e;
  dim3 grid(a.n_chunks, a.H);
  dqkwg_kernel<DK, DV><<<grid, NTHREADS, S::bytes, st>>>(a);
  return check_launch("dqkwg");
}

}  // namespace

int launch_dqkwg(const b200gdn_chunk_args& a, cudaStream_t st) {
  if (a.HV > a.H && a.dq_acc == nullptr) return set_error(B200GDN_ERR_BAD_ARGUMENT, "dqkwg: dq_acc is required when HV > H");
  if (a.K == 128 && a.V == 128) return launch<128, 128>(a, st);
  if (a.K == 64 && a.V == 64) return launch<64, 64>(a, st);
  return set_error(B200GDN_ERR_UNSUPPORTED, "dqkwg: K=%d V=%d not built (64/64 and 128/128 are)", a.K, a.V);
}

}  // namespace gdn
