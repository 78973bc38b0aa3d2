// Intra-chunk part of the value gradient:
//     dv_local[j] = sum_{i >= j} scale <k_j, q_i> 2^(gamma_i - gamma_j) do_i
// Replaces chunk_bwd_kernel_dv_local (fla/ops/common/chunk_o.py:465-540).  One CTA per (chunk, value
// head); the result is written into the dv2 buffer, which the reverse scan then completes in place.
#include "gdn_common.cuh"

namespace gdn {
namespace {

constexpr int NTHREADS = 128;

template <int DK, int DV>
struct DvSmem {
  static constexpr int LDK = DK + PAD, LDV = DV + PAD, LDP = BT + PAD;
  static constexpr size_t q_off = 0;
  static constexpr size_t k_off = q_off + sizeof(__nv_bfloat16) * BT * LDK;
  static constexpr size_t d_off = k_off + sizeof(__nv_bfloat16) * BT * LDK;
  static constexpr size_t p_off = d_off + sizeof(__nv_bfloat16) * BT * LDV;
  static constexpr size_t g_off = p_off + sizeof(__nv_bfloat16) * BT * LDP;
  static constexpr size_t bytes = g_off + sizeof(float) * BT;
  static_assert(2 * BT * LDK >= BT * LDV, "output staging fits in the q/k tiles");
};

template <int DK, int DV>
__global__ void __launch_bounds__(NTHREADS) dv_local_kernel(const b200gdn_chunk_args a) {
  using S = DvSmem<DK, DV>;
  extern __shared__ __align__(16) unsigned char smem[];
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem + S::q_off);
  __nv_bfloat16* Ks = reinterpret_cast<__nv_bfloat16*>(smem + S::k_off);
  __nv_bfloat16* Ds = reinterpret_cast<__nv_bfloat16*>(smem + S::d_off);
  __nv_bfloat16* Ps = reinterpret_cast<__nv_bfloat16*>(smem + S::p_off);
  float* gs = reinterpret_cast<float*>(smem + S::g_off);
  __nv_bfloat16* stage = Qs;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int c = blockIdx.x, hv = blockIdx.y;
  const int G = a.HV / a.H, hq = hv / G;
  const ChunkMeta cm = load_chunk_meta(a.chunk_meta, c);
  const int64_t row0 = cm.row;

  load_tile_async<DK, NTHREADS>(Qs, reinterpret_cast<const __nv_bfloat16*>(a.q) + (row0 * a.H + hq) * DK,
                                (int64_t)a.H * DK, cm.len, tid);
  load_tile_async<DK, NTHREADS>(Ks, reinterpret_cast<const __nv_bfloat16*>(a.k) + (row0 * a.H + hq) * DK,
                                (int64_t)a.H * DK, cm.len, tid);
  load_tile_async<DV, NTHREADS>(Ds, reinterpret_cast<const __nv_bfloat16*>(a.d_o) + (row0 * a.HV + hv) * DV,
                                (int64_t)a.HV * DV, cm.len, tid);
  cp_async_commit();
  load_gamma(gs, a.gamma, c, a.HV, hv, tid);
  cp_async_wait<0>();
  __syncthreads();

  // P[i][j] = scale (q_i . k_j) 2^(gamma_i - gamma_j) for i >= j, stored row-major in shared memory
  {
    float acc[8][4];
    zero_acc<8>(acc);
    warp_mma<8, DK / 16, AMajor::Row, BMajor::NK>(acc, Qs + warp * 16 * S::LDK, S::LDK, Ks, S::LDK, lane);
    const int r_lo = warp * 16 + g, r_hi = r_lo + 8;
    const float g_lo = gs[r_lo], g_hi = gs[r_hi];
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        int i = (e & 2) ? r_hi : r_lo;
        int j = nt * 8 + 2 * t + (e & 1);
        float gi = (e & 2) ? g_hi : g_lo;
        acc[nt][e] = (i >= j) ? acc[nt][e] * a.scale * exp2f(gi - gs[j]) : 0.f;
      }
    }
    acc_to_smem<8>(Ps + warp * 16 * S::LDP, S::LDP, acc, lane);
  }
  __syncthreads();

  // dv_local = P^T do   (rows j = warp*16.., contraction over i)
  float dv[DV / 8][4];
  zero_acc<DV / 8>(dv);
  warp_mma<DV / 8, BT / 16, AMajor::Trans, BMajor::KN>(dv, Ps + warp * 16, S::LDP, Ds, S::LDV, lane);
  __syncthreads();
  acc_to_smem<DV / 8>(stage + warp * 16 * S::LDV, S::LDV, dv, lane);
  __syncthreads();
  store_tile<BT, DV, NTHREADS>(reinterpret_cast<__nv_bfloat16*>(a.dv2) + (row0 * a.HV + hv) * DV, (int64_t)a.HV * DV,
                               stage, cm.len, tid);
}

template <int DK, int DV>
int launch(const b200gdn_chunk_args& a, cudaStream_t st) {
  using S = DvSmem<DK, DV>;
  if (int e = ensure_smem(dv_local_kernel<DK, DV>, S::bytes)) return e;
  dim3 grid(a.n_chunks, a.HV);
  dv_local_kernel<DK, DV><<<grid, NTHREADS, S::bytes, st>>>(a);
  return check_launch("dv_local");
}

}  // namespace

int launch_dv_local(const b200gdn_chunk_args& a, cudaStream_t st) {
  if (a.K == 128 && a.V == 128) return launch<128, 128>(a, st);
  if (a.K == 64 && a.V == 64) return launch<64, 64>(a, st);
  return set_error(B200GDN_ERR_UNSUPPORTED, "dv_local: K=%d V=%d not built (64/64 and 128/128 are)", a.K, a.V);
}

}  // namespace gdn
