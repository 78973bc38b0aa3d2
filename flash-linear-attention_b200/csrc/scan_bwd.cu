// Reverse state-gradient scan: for every (sequence, value head) walk the chunks backwards with the
// K x V gradient dS resident in registers:
//     dh_c = dS (bf16 snapshot, gradient w.r.t. the state at chunk END)
//     dv2  = (K dS) 2^(gamma_last - gamma) + dv_local
//     dS  <- 2^gamma_last dS + scale (Q 2^gamma)^T do - W^T dv2
// Replaces chunk_gated_delta_rule_bwd_kernel_dhu_blockdim64 (fla/ops/common/chunk_delta_h.py:369-683).
// Same CTA layout as the forward scan (a BV-wide column slice per CTA, warps 4 x BV/32).
//
// With d_o == NULL (zeros), dv2 initialised to zeros, dht = identity and V := K the result in dh0 is the
// backward transition matrix of a shard for context parallelism (fla/ops/cp/chunk_delta_h.py:478-744).
#include "gdn_common.cuh"

namespace gdn {
namespace {

template <int DK, int BV>
struct ScanBwdSmem {
  static constexpr int LDK = DK + PAD, LDB = BV + PAD;
  static constexpr size_t t_bytes = sizeof(__nv_bfloat16) * BT * LDK;
  static constexpr size_t s_bytes = sizeof(__nv_bfloat16) * BT * LDB;
  static constexpr size_t stage_bytes = 3 * t_bytes + 2 * s_bytes + sizeof(float) * BT;  // Q, K, W, do, dv_local, gamma
  static constexpr size_t sb_off = 2 * stage_bytes;
  static constexpr size_t bytes = sb_off + sizeof(__nv_bfloat16) * DK * LDB;
};

template <int DK, int DV, int BV>
__global__ void __launch_bounds__(128 * (BV / 32)) scan_bwd_kernel(const b200gdn_chunk_args a) {
  constexpr int NCG = BV / 32;
  constexpr int NTHREADS = 128 * NCG;
  constexpr int MT = DK / 64;
  using S = ScanBwdSmem<DK, BV>;
  extern __shared__ __align__(16) unsigned char smem[];
  __nv_bfloat16* Sb = reinterpret_cast<__nv_bfloat16*>(smem + S::sb_off);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int rg = warp & 3, cg = warp >> 2;
  const int g = lane >> 2, t = lane & 3;
  const int v0 = blockIdx.x * BV, hv = blockIdx.y, n = blockIdx.z;
  const int G = a.HV / a.H, hq = hv / G;
  const int c_first = a.seq_meta[2 * n], nc = a.seq_meta[2 * n + 1];

  const __nv_bfloat16* qbase = reinterpret_cast<const __nv_bfloat16*>(a.q);
  const __nv_bfloat16* kbase = reinterpret_cast<const __nv_bfloat16*>(a.k);
  const __nv_bfloat16* wbase = reinterpret_cast<const __nv_bfloat16*>(a.w);
  const __nv_bfloat16* dobase = reinterpret_cast<const __nv_bfloat16*>(a.d_o);
  __nv_bfloat16* dv2base = reinterpret_cast<__nv_bfloat16*>(a.dv2);

  auto issue_loads = [&](const ChunkMeta& cm, int c, int s) {
    unsigned char* base = smem + (size_t)s * S::stage_bytes;
    __nv_bfloat16* Qt = reinterpret_cast<__nv_bfloat16*>(base);
    __nv_bfloat16* Kt = reinterpret_cast<__nv_bfloat16*>(base + S::t_bytes);
    __nv_bfloat16* Wt = reinterpret_cast<__nv_bfloat16*>(base + 2 * S::t_bytes);
    __nv_bfloat16* Dt = reinterpret_cast<__nv_bfloat16*>(base + 3 * S::t_bytes);
    __nv_bfloat16* Lt = reinterpret_cast<__nv_bfloat16*>(base + 3 * S::t_bytes + S::s_bytes);
    float* gs = reinterpret_cast<float*>(base + 3 * S::t_bytes + 2 * S::s_bytes);
    load_tile_async<DK, NTHREADS>(Qt, qbase + ((int64_t)cm.row * a.H + hq) * DK, (int64_t)a.H * DK, cm.len, tid);
    load_tile_async<DK, NTHREADS>(Kt, kbase + ((int64_t)cm.row * a.H + hq) * DK, (int64_t)a.H * DK, cm.len, tid);
    load_tile_async<DK, NTHREADS>(Wt, wbase + ((int64_t)cm.row * a.HV + hv) * DK, (int64_t)a.HV * DK, cm.len, tid);
    if (dobase != nullptr)
      load_tile_async<BV, NTHREADS>(Dt, dobase + ((int64_t)cm.row * a.HV + hv) * DV + v0, (int64_t)a.HV * DV, cm.len, tid);
    load_tile_async<BV, NTHREADS>(Lt, dv2base + ((int64_t)cm.row * a.HV + hv) * DV + v0, (int64_t)a.HV * DV, cm.len, tid);
    load_gamma_async(gs, a.gamma, c, a.HV, hv, tid);
  };

  float S_[MT][4][4];
  {
    const float* dht = a.dht ? a.dht + ((int64_t)n * a.HV + hv) * DK * DV : nullptr;
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int nt = 0; nt < 4; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          int r = rg * (DK / 4) + mt * 16 + g + ((e >> 1) << 3);
          int col = v0 + cg * 32 + nt * 8 + 2 * t + (e & 1);
          S_[mt][nt][e] = dht ? dht[(int64_t)r * DV + col] : 0.f;
        }
  }

  // chunk descriptors are fetched two iterations ahead so that no global-load latency sits on the chain
  const int c_last = c_first + nc - 1;
  ChunkMeta cm_cur = load_chunk_meta(a.chunk_meta, nc > 0 ? c_last : c_first);
  ChunkMeta cm_nxt = load_chunk_meta(a.chunk_meta, nc > 1 ? c_last - 1 : c_first);
  if (nc > 0) issue_loads(cm_cur, c_last, 0);
  cp_async_commit();

  for (int ic = 0; ic < nc; ++ic) {
    const int c = c_last - ic, s = ic & 1;
    const ChunkMeta cm = cm_cur;
    const ChunkMeta cm_nn = load_chunk_meta(a.chunk_meta, ic + 2 < nc ? c - 2 : c);
    unsigned char* base = smem + (size_t)s * S::stage_bytes;
    const __nv_bfloat16* Qt = reinterpret_cast<const __nv_bfloat16*>(base);
    const __nv_bfloat16* Kt = reinterpret_cast<const __nv_bfloat16*>(base + S::t_bytes);
    const __nv_bfloat16* Wt = reinterpret_cast<const __nv_bfloat16*>(base + 2 * S::t_bytes);
    __nv_bfloat16* Dt = reinterpret_cast<__nv_bfloat16*>(base + 3 * S::t_bytes);
    __nv_bfloat16* Lt = reinterpret_cast<__nv_bfloat16*>(base + 3 * S::t_bytes + S::s_bytes);
    const float* gs = reinterpret_cast<const float*>(base + 3 * S::t_bytes + 2 * S::s_bytes);

    cp_async_wait<0>();
    __syncthreads();
    if (ic + 1 < nc) issue_loads(cm_nxt, c - 1, s ^ 1);
    cp_async_commit();
    cm_cur = cm_nxt;
    cm_nxt = cm_nn;

#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
      acc_to_smem<4>(Sb + (rg * (DK / 4) + mt * 16) * S::LDB + cg * 32, S::LDB, S_[mt], lane);
    __syncthreads();
    if (a.dh != nullptr) {
      __nv_bfloat16* hg = reinterpret_cast<__nv_bfloat16*>(a.dh) + ((int64_t)c * a.HV + hv) * DK * DV + v0;
      store_tile<DK, BV, NTHREADS>(hg, DV, Sb, DK, tid);
    }

    // dv2 = (K dS) 2^(gamma_last - gamma) + dv_local ; in place over the dv_local slice.
    // do <- do * scale * 2^gamma in place (the right-hand side of the Q^T product).
    float acc[4][4];
    zero_acc<4>(acc);
    warp_mma<4, DK / 16, AMajor::Row, BMajor::KN>(acc, Kt + rg * 16 * S::LDK, S::LDK, Sb + cg * 32, S::LDB, lane);
    const float glast = gs[BT - 1];
    {
      const int r_lo = rg * 16 + g, r_hi = r_lo + 8;
      const float e_lo = exp2f(glast - gs[r_lo]), e_hi = exp2f(glast - gs[r_hi]);
      const float q_lo = a.scale * exp2f(gs[r_lo]), q_hi = a.scale * exp2f(gs[r_hi]);
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
        const int col = cg * 32 + nt * 8 + 2 * t;
        uint32_t* pl_lo = reinterpret_cast<uint32_t*>(Lt + r_lo * S::LDB + col);
        uint32_t* pl_hi = reinterpret_cast<uint32_t*>(Lt + r_hi * S::LDB + col);
        float2 l_lo = unpack_bf16(*pl_lo), l_hi = unpack_bf16(*pl_hi);
        *pl_lo = pack_bf16(acc[nt][0] * e_lo + l_lo.x, acc[nt][1] * e_lo + l_lo.y);
        *pl_hi = pack_bf16(acc[nt][2] * e_hi + l_hi.x, acc[nt][3] * e_hi + l_hi.y);
        uint32_t* pd_lo = reinterpret_cast<uint32_t*>(Dt + r_lo * S::LDB + col);
        uint32_t* pd_hi = reinterpret_cast<uint32_t*>(Dt + r_hi * S::LDB + col);
        if (dobase != nullptr) {
          float2 d_lo = unpack_bf16(*pd_lo), d_hi = unpack_bf16(*pd_hi);
          *pd_lo = pack_bf16(d_lo.x * q_lo, d_lo.y * q_lo);
          *pd_hi = pack_bf16(d_hi.x * q_hi, d_hi.y * q_hi);
        }
      }
    }
    __syncthreads();
    store_tile<BT, BV, NTHREADS>(dv2base + ((int64_t)cm.row * a.HV + hv) * DV + v0, (int64_t)a.HV * DV, Lt, cm.len, tid);

    // dS <- 2^gamma_last dS + Q^T (do scale 2^gamma) - W^T dv2
    const float dec = exp2f(glast);
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
      for (int nt = 0; nt < 4; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) S_[mt][nt][e] *= dec;
      if (dobase != nullptr)
        warp_mma<4, BT / 16, AMajor::Trans, BMajor::KN>(S_[mt], Qt + rg * (DK / 4) + mt * 16, S::LDK, Dt + cg * 32,
                                                        S::LDB, lane);
      warp_mma<4, BT / 16, AMajor::Trans, BMajor::KN, true>(S_[mt], Wt + rg * (DK / 4) + mt * 16, S::LDK, Lt + cg * 32,
                                                            S::LDB, lane);
    }
  }

  if (a.dh0 != nullptr) {
    float* d0 = a.dh0 + ((int64_t)n * a.HV + hv) * DK * DV;
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
        int r = rg * (DK / 4) + mt * 16 + g;
        int col = v0 + cg * 32 + nt * 8 + 2 * t;
        *reinterpret_cast<float2*>(&d0[(int64_t)r * DV + col]) = make_float2(S_[mt][nt][0], S_[mt][nt][1]);
        *reinterpret_cast<float2*>(&d0[(int64_t)(r + 8) * DV + col]) = make_float2(S_[mt][nt][2], S_[mt][nt][3]);
      }
  }
}

template <int DK, int DV, int BV>
int launch(const b200gdn_chunk_args& a, cudaStream_t st) {
  using S = ScanBwdSmem<DK, BV>;
  if (int e = ensure_smem(scan_bwd_kernel<DK, DV, BV>, S::bytes)) return e;
  dim3 grid(DV / BV, a.HV, a.n_seq);
  scan_bwd_kernel<DK, DV, BV><<<grid, 128 * (BV / 32), S::bytes, st>>>(a);
  return check_launch("scan_bwd");
}

}  // namespace

int launch_scan_bwd(const b200gdn_chunk_args& a, cudaStream_t st) {
  if (a.K == 128 && a.V == 128) return launch<128, 128, 64>(a, st);
  if (a.K == 64 && a.V == 64) return launch<64, 64, 32>(a, st);
  return set_error(B200GDN_ERR_UNSUPPORTED, "scan_bwd: K=%d V=%d not built (64/64 and 128/128 are)", a.K, a.V);
}

}  // namespace gdn
