// Forward state scan: for every (sequence, value head) walk the chunks in order with the K x V state
// resident in registers (fp32 accumulator fragments):
//     h_c = S (bf16 snapshot, state at chunk start);  v_new = U - W S;
//     S <- 2^gamma_last S + (K 2^(gamma_last - gamma))^T v_new.
// Replaces chunk_gated_delta_rule_fwd_kernel_h_blockdim64 (fla/ops/common/chunk_delta_h.py:58-348).
//
// One CTA owns a BV-wide column slice of one state: warps are laid out 4 (row groups of K/4... of the
// state, 16-row groups of the chunk) x BV/32 (column groups of 32), so the W and K tiles are loaded
// once per CTA and shared by all column groups.  Loads of chunk c+1 (cp.async) overlap the two
// dependent contractions of chunk c.
//
// The same kernel produces the transition matrix of a whole shard for context parallelism
// (fla/ops/cp/chunk_delta_h.py:254-315): with u == NULL (zeros), h0 = identity and V := K the final
// state is M = prod_c (2^gamma_last I - K~^T W).
#include "gdn_common.cuh"

namespace gdn {
namespace {

template <int DK, int BV, int NSTAGE>
struct ScanFwdSmem {
  static constexpr int LDK = DK + PAD, LDB = BV + PAD;
  static constexpr size_t w_bytes = sizeof(__nv_bfloat16) * BT * LDK;
  static constexpr size_t u_bytes = sizeof(__nv_bfloat16) * BT * LDB;
  static constexpr size_t stage_bytes = 2 * w_bytes + u_bytes + sizeof(float) * BT;  // W, K, U-slice, gamma
  static constexpr size_t sb_off = NSTAGE * stage_bytes;                                   // bf16 state [DK][LDB]
  static constexpr size_t vn_off = sb_off + sizeof(__nv_bfloat16) * DK * LDB;         // bf16 v_new slice
  static constexpr size_t vt_off = vn_off + u_bytes;                                  // bf16 gated v_new slice
  static constexpr size_t bytes = vt_off + u_bytes;
};

template <int DK, int DV, int BV, int NSTAGE, int CW>
__global__ void __launch_bounds__(128 * (BV / CW)) scan_fwd_kernel(const b200gdn_chunk_args a) {
  constexpr int NCG = BV / CW;          // column groups of CW columns
  constexpr int NT = CW / 8;            // n-tiles per warp
  constexpr int NTHREADS = 128 * NCG;
  constexpr int MT = DK / 64;           // 16-row m-tiles of the state per warp (4 row groups)
  using S = ScanFwdSmem<DK, BV, NSTAGE>;
  extern __shared__ __align__(16) unsigned char smem[];
  __nv_bfloat16* Sb = reinterpret_cast<__nv_bfloat16*>(smem + S::sb_off);
  __nv_bfloat16* Vn = reinterpret_cast<__nv_bfloat16*>(smem + S::vn_off);
  __nv_bfloat16* Vt = reinterpret_cast<__nv_bfloat16*>(smem + S::vt_off);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int rg = warp & 3, cg = warp >> 2;
  const int g = lane >> 2, t = lane & 3;
  const int v0 = blockIdx.x * BV, hv = blockIdx.y, n = blockIdx.z;
  const int G = a.HV / a.H, hq = hv / G;
  const int c_first = a.seq_meta[2 * n], nc = a.seq_meta[2 * n + 1];

  const __nv_bfloat16* kbase = reinterpret_cast<const __nv_bfloat16*>(a.k);
  const __nv_bfloat16* wbase = reinterpret_cast<const __nv_bfloat16*>(a.w);
  const __nv_bfloat16* ubase = reinterpret_cast<const __nv_bfloat16*>(a.u);

  auto stage_ptr = [&](int s) { return smem + (size_t)s * S::stage_bytes; };
  auto issue_loads = [&](const ChunkMeta& cm, int s) {
    unsigned char* base = stage_ptr(s);
    __nv_bfloat16* Wt = reinterpret_cast<__nv_bfloat16*>(base);
    __nv_bfloat16* Kt = reinterpret_cast<__nv_bfloat16*>(base + S::w_bytes);
    __nv_bfloat16* Ut = reinterpret_cast<__nv_bfloat16*>(base + 2 * S::w_bytes);
    float* gs = reinterpret_cast<float*>(base + 2 * S::w_bytes + S::u_bytes);
    load_tile_async<DK, NTHREADS>(Wt, wbase + ((int64_t)cm.row * a.HV + hv) * DK, (int64_t)a.HV * DK, cm.len, tid);
    load_tile_async<DK, NTHREADS>(Kt, kbase + ((int64_t)cm.row * a.H + hq) * DK, (int64_t)a.H * DK, cm.len, tid);
    if (ubase != nullptr)
      load_tile_async<BV, NTHREADS>(Ut, ubase + ((int64_t)cm.row * a.HV + hv) * DV + v0, (int64_t)a.HV * DV, cm.len, tid);
    load_gamma_async(gs, a.gamma, cm.row, cm.len, a.HV, hv, tid);
  };

  // state fragments: rows rg*(DK/4) + mt*16 + {g, g+8}, columns cg*32 + nt*8 + 2t + {0,1}
  float S_[MT][NT][4];
  {
    const float* h0 = a.h0 ? a.h0 + ((int64_t)n * a.HV + hv) * DK * DV : nullptr;
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          int r = rg * (DK / 4) + mt * 16 + g + ((e >> 1) << 3);
          int col = v0 + cg * CW + nt * 8 + 2 * t + (e & 1);
          S_[mt][nt][e] = h0 ? h0[(int64_t)r * DV + col] : 0.f;
        }
  }

  // NSTAGE-deep prefetch: the tiles of chunk ic + NSTAGE - 1 are requested while chunk ic is processed, so
  // neither the tile loads nor the chunk descriptors they depend on sit on the recurrence's critical path.
  ChunkMeta cm_q[NSTAGE];
#pragma unroll
  for (int s = 0; s < NSTAGE; ++s) cm_q[s] = load_chunk_meta(a.chunk_meta, c_first + (s < nc ? s : 0));
#pragma unroll
  for (int s = 0; s < NSTAGE - 1; ++s) {
    if (s < nc) issue_loads(cm_q[s], s);
    cp_async_commit();
  }

  for (int ic = 0; ic < nc; ++ic) {
    const int c = c_first + ic, s = ic % NSTAGE;
    const ChunkMeta cm = cm_q[0];
    const ChunkMeta cm_far = load_chunk_meta(a.chunk_meta, c_first + (ic + NSTAGE < nc ? ic + NSTAGE : ic));
    unsigned char* base = stage_ptr(s);
    const __nv_bfloat16* Wt = reinterpret_cast<const __nv_bfloat16*>(base);
    const __nv_bfloat16* Kt = reinterpret_cast<const __nv_bfloat16*>(base + S::w_bytes);
    const __nv_bfloat16* Ut = reinterpret_cast<const __nv_bfloat16*>(base + 2 * S::w_bytes);
    const float* gs = reinterpret_cast<const float*>(base + 2 * S::w_bytes + S::u_bytes);

    cp_async_wait<NSTAGE - 2>();
    __syncthreads();  // stage s landed; every warp is done with the previous chunk (its stage, Sb, Vt)
    if (ic + NSTAGE - 1 < nc) issue_loads(cm_q[NSTAGE - 1], (ic + NSTAGE - 1) % NSTAGE);
    cp_async_commit();
#pragma unroll
    for (int q = 0; q < NSTAGE - 1; ++q) cm_q[q] = cm_q[q + 1];
    cm_q[NSTAGE - 1] = cm_far;

    // bf16 snapshot of the state -> shared (operand of W S) and -> global h_c
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
      acc_to_smem<NT>(Sb + (rg * (DK / 4) + mt * 16) * S::LDB + cg * CW, S::LDB, S_[mt], lane);
    __syncthreads();
    if (a.h != nullptr) {
      __nv_bfloat16* hg = reinterpret_cast<__nv_bfloat16*>(a.h) + ((int64_t)c * a.HV + hv) * DK * DV + v0;
      store_tile<DK, BV, NTHREADS>(hg, DV, Sb, DK, tid);
    }

    // v_new = U - W S   (rows rg*16.., columns cg*32..)
    float acc[NT][4];
    zero_acc<NT>(acc);
    warp_mma<NT, DK / 16, AMajor::Row, BMajor::KN>(acc, Wt + rg * 16 * S::LDK, S::LDK, Sb + cg * CW, S::LDB, lane);
    const float glast = gs[BT - 1];
    {
      const int r_lo = rg * 16 + g, r_hi = r_lo + 8;
      const float e_lo = exp2f(glast - gs[r_lo]), e_hi = exp2f(glast - gs[r_hi]);
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        const int col = cg * CW + nt * 8 + 2 * t;
        float2 u_lo = make_float2(0.f, 0.f), u_hi = make_float2(0.f, 0.f);
        if (ubase != nullptr) {
          u_lo = unpack_bf16(*reinterpret_cast<const uint32_t*>(Ut + r_lo * S::LDB + col));
          u_hi = unpack_bf16(*reinterpret_cast<const uint32_t*>(Ut + r_hi * S::LDB + col));
        }
        float v00 = u_lo.x - acc[nt][0], v01 = u_lo.y - acc[nt][1];
        float v10 = u_hi.x - acc[nt][2], v11 = u_hi.y - acc[nt][3];
        *reinterpret_cast<uint32_t*>(Vn + r_lo * S::LDB + col) = pack_bf16(v00, v01);
        *reinterpret_cast<uint32_t*>(Vn + r_hi * S::LDB + col) = pack_bf16(v10, v11);
        *reinterpret_cast<uint32_t*>(Vt + r_lo * S::LDB + col) = pack_bf16(v00 * e_lo, v01 * e_lo);
        *reinterpret_cast<uint32_t*>(Vt + r_hi * S::LDB + col) = pack_bf16(v10 * e_hi, v11 * e_hi);
      }
    }
    __syncthreads();
    if (a.v_new != nullptr) {
      __nv_bfloat16* vg = reinterpret_cast<__nv_bfloat16*>(a.v_new) + ((int64_t)cm.row * a.HV + hv) * DV + v0;
      store_tile<BT, BV, NTHREADS>(vg, (int64_t)a.HV * DV, Vn, cm.len, tid);
    }

    // S <- 2^gamma_last S + K^T v~     (rows rg*(DK/4) + mt*16.., columns cg*32..)
    const float dec = exp2f(glast);
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) S_[mt][nt][e] *= dec;
      warp_mma<NT, BT / 16, AMajor::Trans, BMajor::KN>(S_[mt], Kt + rg * (DK / 4) + mt * 16, S::LDK, Vt + cg * CW, S::LDB,
                                                      lane);
    }
  }

  if (a.ht != nullptr) {
    float* ht = a.ht + ((int64_t)n * a.HV + hv) * DK * DV;
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        int r = rg * (DK / 4) + mt * 16 + g;
        int col = v0 + cg * CW + nt * 8 + 2 * t;
        *reinterpret_cast<float2*>(&ht[(int64_t)r * DV + col]) = make_float2(S_[mt][nt][0], S_[mt][nt][1]);
        *reinterpret_cast<float2*>(&ht[(int64_t)(r + 8) * DV + col]) = make_float2(S_[mt][nt][2], S_[mt][nt][3]);
      }
  }
}

template <int DK, int DV, int BV, int NSTAGE, int CW>
int launch(const b200gdn_chunk_args& a, cudaStream_t st) {
  using S = ScanFwdSmem<DK, BV, NSTAGE>;
  if (int e = ensure_smem(scan_fwd_kernel<DK, DV, BV, NSTAGE, CW>, S::bytes)) return e;
  dim3 grid(DV / BV, a.HV, a.n_seq);
  scan_fwd_kernel<DK, DV, BV, NSTAGE, CW><<<grid, 128 * (BV / CW), S::bytes, st>>>(a);
  return check_launch("scan_fwd");
}

}  // namespace

int launch_scan_fwd(const b200gdn_chunk_args& a, cudaStream_t st) {
  if (a.K == 128 && a.V == 128) return launch<128, 128, 64, 2, 32>(a, st);
  if (a.K == 64 && a.V == 64) return launch<64, 64, 32, 2, 32>(a, st);
  return set_error(B200GDN_ERR_UNSUPPORTED, "scan_fwd: K=%d V=%d not built (64/64 and 128/128 are)", a.K, a.V);
}

}  // namespace gdn
