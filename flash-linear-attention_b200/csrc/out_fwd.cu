// Chunk output:  o = scale [ (Q h_c) 2^gamma + tril(Q K^T 2^(gamma_i - gamma_j)) v_new ].
// Replaces chunk_fwd_kernel_o (fla/ops/common/chunk_o.py:56-153).  One CTA per (chunk, value head);
// the masked score tile never leaves registers: the accumulator of Q K^T is re-packed as the A operand
// of the product with v_new.
#include "gdn_common.cuh"

namespace gdn {
namespace {

constexpr int NTHREADS = 128;

template <int DK, int DV>
struct OutSmem {
  static constexpr int LDK = DK + PAD, LDV = DV + PAD;
  static constexpr size_t q_off = 0;
  static constexpr size_t k_off = q_off + sizeof(__nv_bfloat16) * BT * LDK;
  static constexpr size_t v_off = k_off + sizeof(__nv_bfloat16) * BT * LDK;
  static constexpr size_t h_off = v_off + sizeof(__nv_bfloat16) * BT * LDV;
  static constexpr size_t g_off = h_off + sizeof(__nv_bfloat16) * DK * LDV;
  static constexpr size_t bytes = g_off + sizeof(float) * BT;
  static_assert(2 * BT * LDK >= BT * LDV, "output staging fits in the q/k tiles");
};

template <int DK, int DV>
__global__ void __launch_bounds__(NTHREADS) out_fwd_kernel(const b200gdn_chunk_args a) {
  using S = OutSmem<DK, DV>;
  extern __shared__ __align__(16) unsigned char smem[];
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem + S::q_off);
  __nv_bfloat16* Ks = reinterpret_cast<__nv_bfloat16*>(smem + S::k_off);
  __nv_bfloat16* Vn = reinterpret_cast<__nv_bfloat16*>(smem + S::v_off);
  __nv_bfloat16* Hs = reinterpret_cast<__nv_bfloat16*>(smem + S::h_off);
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
  load_tile_async<DV, NTHREADS>(Vn, reinterpret_cast<const __nv_bfloat16*>(a.v_new) + (row0 * a.HV + hv) * DV,
                                (int64_t)a.HV * DV, cm.len, tid);
  load_rows_async<DK, DV, NTHREADS>(Hs, reinterpret_cast<const __nv_bfloat16*>(a.h) + ((int64_t)c * a.HV + hv) * DK * DV,
                                    DV, tid);
  cp_async_commit();
  load_gamma(gs, a.gamma, c, a.HV, hv, tid);
  cp_async_wait<0>();
  __syncthreads();

  const int r_lo = warp * 16 + g, r_hi = r_lo + 8;
  const float g_lo = gs[r_lo], g_hi = gs[r_hi];

  // P = tril(Q K^T 2^(gamma_i - gamma_j)), kept as A fragments
  uint32_t pfrag[4][4];
  {
    float acc[8][4];
    zero_acc<8>(acc);
    warp_mma<8, DK / 16, AMajor::Row, BMajor::NK>(acc, Qs + warp * 16 * S::LDK, S::LDK, Ks, S::LDK, lane);
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        int i = (e & 2) ? r_hi : r_lo;
        int j = nt * 8 + 2 * t + (e & 1);
        float gi = (e & 2) ? g_hi : g_lo;
        acc[nt][e] = (i >= j) ? acc[nt][e] * exp2f(gi - gs[j]) : 0.f;
      }
    }
    acc_to_afrag<8>(pfrag, acc);
  }

  float o[DV / 8][4];
  zero_acc<DV / 8>(o);
  warp_mma<DV / 8, DK / 16, AMajor::Row, BMajor::KN>(o, Qs + warp * 16 * S::LDK, S::LDK, Hs, S::LDV, lane);
  {
    const float e_lo = exp2f(g_lo), e_hi = exp2f(g_hi);
#pragma unroll
    for (int nt = 0; nt < DV / 8; ++nt) {
      o[nt][0] *= e_lo; o[nt][1] *= e_lo; o[nt][2] *= e_hi; o[nt][3] *= e_hi;
    }
  }
  warp_mma_ra<DV / 8, 4, BMajor::KN>(o, pfrag, Vn, S::LDV, lane);
#pragma unroll
  for (int nt = 0; nt < DV / 8; ++nt) {
    o[nt][0] *= a.scale; o[nt][1] *= a.scale; o[nt][2] *= a.scale; o[nt][3] *= a.scale;
  }
  __syncthreads();  // every warp is done reading Qs/Ks before they become the staging tile
  acc_to_smem<DV / 8>(stage + warp * 16 * S::LDV, S::LDV, o, lane);
  __syncthreads();
  store_tile<BT, DV, NTHREADS>(reinterpret_cast<__nv_bfloat16*>(a.o) + (row0 * a.HV + hv) * DV, (int64_t)a.HV * DV, stage,
                               cm.len, tid);
}

template <int DK, int DV>
int launch(const b200gdn_chunk_args& a, cudaStream_t st) {
  using S = OutSmem<DK, DV>;
  if (int e = ensure_smem(out_fwd_kernel<DK, DV>, S::bytes)) return e;
  dim3 grid(a.n_chunks, a.HV);
  out_fwd_kernel<DK, DV><<<grid, NTHREADS, S::bytes, st>>>(a);
  return check_launch("out_fwd");
}

}  // namespace

int launch_out_fwd(const b200gdn_chunk_args& a, cudaStream_t st) {
  if (a.K == 128 && a.V == 128) return launch<128, 128>(a, st);
  if (a.K == 64 && a.V == 64) return launch<64, 64>(a, st);
  return set_error(B200GDN_ERR_UNSUPPORTED, "out_fwd: K=%d V=%d not built (64/64 and 128/128 are)", a.K, a.V);
}

}  // namespace gdn
