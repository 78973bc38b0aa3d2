// Forward state scan: for every (sequence, value head) walk the chunks in order with the K x V state
// resident on chip (fp32 accumulator fragments in registers):
//     h_c = S (bf16 snapshot, state at chunk start);  v_new = U - W S;
//     S <- 2^gamma_last S + (K 2^(gamma_last - gamma))^T v_new.
// Replaces chunk_gated_delta_rule_fwd_kernel_h_blockdim64 (fla/ops/common/chunk_delta_h.py:58-348).
//
// The recurrence is a chain of 64-row steps, so what matters is the latency of one step.  Global-memory
// instructions issued by the compute warps used to dominate it, therefore data movement is taken off
// those warps entirely:
//   * a producer warp feeds a ring of NSTAGE stages with TMA (cp.async.bulk.tensor, 128-byte swizzle):
//     W [64 x K], K [64 x K] and the U slice [64 x 64] of chunk c + NSTAGE - 1 are in flight while chunk
//     c is processed; full/empty mbarriers hand the stages over;
//   * eight compute warps (4 row groups x 2 column groups of one 64-column slice of the state) run the
//     two dependent contractions with mma.sync from the swizzled tiles;
//   * the bf16 state snapshot h_c and v_new leave through TMA stores from double-buffered shared tiles.
// A ragged last chunk is loaded as a full box (rows of the next sequence or zero fill); its extra rows
// are masked where v_new is formed, and its v_new rows are written with plain predicated stores.
//
// The same kernel produces the transition matrix of a whole shard for context parallelism
// (fla/ops/cp/chunk_delta_h.py:254-315): with u == NULL (zeros), h0 = identity and V := K the final
// state is M = prod_c (2^gamma_last I - K~^T W).
#include "gdn_common.cuh"
#include "tc5.cuh"
#include "tma.cuh"

namespace gdn {
namespace {

constexpr int BV = 64;            // state columns per CTA
constexpr int NCOMPUTE = 256;     // 8 compute warps
constexpr int NTHREADS = NCOMPUTE + 32;
__device__ int g_scan_fwd_timeout = 0;

template <int DK, int NSTAGE>
struct ScanFwdSmem {
  static constexpr size_t w_bytes = BT * DK * 2;            // W tile, K tile
  static constexpr size_t u_bytes = BT * BV * 2;
  static constexpr size_t stage_bytes = 2 * w_bytes + u_bytes;
  static constexpr size_t o_sb = NSTAGE * stage_bytes;      // 2 x state snapshot [DK][64]
  static constexpr size_t sb_bytes = DK * BV * 2;
  static constexpr size_t o_vn = o_sb + 2 * sb_bytes;       // 2 x v_new slice [64][64]
  static constexpr size_t o_vt = o_vn + 2 * u_bytes;        // gated v_new slice
  static constexpr size_t o_gam = o_vt + u_bytes;           // NSTAGE x 64 floats
  static constexpr size_t o_bar = o_gam + NSTAGE * BT * 4;
  static constexpr size_t bytes = o_bar + 2 * NSTAGE * 8 + 1024;  // + alignment slack
};

struct ScanFwdMaps {
  CUtensorMap w, k, u, h, vn;
};

__device__ __forceinline__ void bar_compute(int id) { asm volatile("bar.sync %0, %1;\n" ::"r"(id), "n"(NCOMPUTE) : "memory"); }

template <int DK, int DV, int NSTAGE>
__global__ void __launch_bounds__(NTHREADS) scan_fwd_kernel(const b200gdn_chunk_args a, const __grid_constant__ ScanFwdMaps maps) {
  using S = ScanFwdSmem<DK, NSTAGE>;
  constexpr int MT = DK / 64;   // 16-row m-tiles of the state per warp
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  float* gam_all = reinterpret_cast<float*>(smem + S::o_gam);
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + S::o_bar);
  uint64_t* empty = full + NSTAGE;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int v0 = blockIdx.x * BV, hv = blockIdx.y, n = blockIdx.z;
  const int G = a.HV / a.H, hq = hv / G;
  const int c_first = a.seq_meta[2 * n], nc = a.seq_meta[2 * n + 1];
  const bool has_u = a.u != nullptr;

  if (tid == 0) {
    for (int s = 0; s < NSTAGE; ++s) {
      tc5::mbar_init(&full[s], 2);               // producer's expect_tx arrive + its gamma arrive
      tc5::mbar_init(&empty[s], NCOMPUTE / 32);  // one arrive per compute warp
    }
    tc5::fence_mbar_init();
  }
  __syncthreads();

  if (warp == NCOMPUTE / 32) {
    // ================= producer warp =================
    if (lane == 0) {
      tma::prefetch_map(&maps.w);
      tma::prefetch_map(&maps.k);
      if (has_u) tma::prefetch_map(&maps.u);
    }
    const uint32_t tx_bytes = (uint32_t)(2 * S::w_bytes + (has_u ? S::u_bytes : 0));
    for (int ic = 0; ic < nc; ++ic) {
      const int s = ic % NSTAGE;
      const ChunkMeta cm = load_chunk_meta(a.chunk_meta, c_first + ic);
      if (ic >= NSTAGE) {
        if (!tc5::mbar_wait(&empty[s], ((ic / NSTAGE) - 1) & 1)) {
          if (lane == 0) atomicExch(&g_scan_fwd_timeout, 1);
          break;
        }
      }
      unsigned char* base = smem + (size_t)s * S::stage_bytes;
      if (lane == 0) {
        tc5::mbar_expect_tx(&full[s], tx_bytes);
#pragma unroll
        for (int p = 0; p < DK / 64; ++p) {
          tma::load_2d(base + p * (BT * 128), &maps.w, hv * DK + p * 64, cm.row, &full[s]);
          tma::load_2d(base + S::w_bytes + p * (BT * 128), &maps.k, hq * DK + p * 64, cm.row, &full[s]);
        }
        if (has_u) tma::load_2d(base + 2 * S::w_bytes, &maps.u, hv * DV + v0, cm.row, &full[s]);
      }
      // gamma of the chunk (rows past the valid length repeat the last valid value)
      float* gs = gam_all + s * BT;
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int i = lane + 32 * j;
        const int r = i < cm.len ? i : cm.len - 1;
        gs[i] = a.gamma[(int64_t)(cm.row + r) * a.HV + hv];
      }
      __syncwarp();
      if (lane == 0) tc5::mbar_arrive(&full[s]);
    }
    return;
  }

  // ================= compute warps =================
  const int rg = warp & 3, cg = warp >> 2;
  const int g = lane >> 2, t = lane & 3;
  const uint32_t sb_base = smem_u32(smem + S::o_sb);
  const uint32_t vn_base = smem_u32(smem + S::o_vn);
  const uint32_t vt_tile = smem_u32(smem + S::o_vt);

  // state fragments: rows rg*(DK/4) + mt*16 + {g, g+8}, columns cg*32 + nt*8 + 2t + {0,1}
  float S_[MT][4][4];
  {
    const float* h0 = a.h0 ? a.h0 + ((int64_t)n * a.HV + hv) * DK * DV : nullptr;
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int nt = 0; nt < 4; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          int r = rg * (DK / 4) + mt * 16 + g + ((e >> 1) << 3);
          int col = v0 + cg * 32 + nt * 8 + 2 * t + (e & 1);
          S_[mt][nt][e] = h0 ? h0[(int64_t)r * DV + col] : 0.f;
        }
  }

  bool failed = false;
  for (int ic = 0; ic < nc; ++ic) {
    const int c = c_first + ic, s = ic % NSTAGE, buf = ic & 1;
    const ChunkMeta cm = load_chunk_meta(a.chunk_meta, c);   // consumed late in the step: latency is hidden
    const uint32_t w_tile = smem_u32(smem + (size_t)s * S::stage_bytes);
    const uint32_t k_tile = w_tile + (uint32_t)S::w_bytes;
    const uint32_t u_tile = w_tile + 2 * (uint32_t)S::w_bytes;
    const float* gs = gam_all + s * BT;
    const uint32_t sb_tile = sb_base + buf * (uint32_t)S::sb_bytes;
    const uint32_t vn_tile = vn_base + buf * (uint32_t)S::u_bytes;

    // bf16 snapshot of the state -> shared (operand of W S, and the source of the h_c store).
    // The buffer was last read two steps ago (contraction) and by the store that thread 0 has waited for.
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) acc_to_swz<4>(sb_tile, DK, rg * (DK / 4) + mt * 16, cg * 32, S_[mt], lane);
    tc5::fence_async_smem();
    if (!tc5::mbar_wait(&full[s], (ic / NSTAGE) & 1)) failed = true;   // tiles of this chunk have landed
    bar_compute(1);
    if (tid == 0 && a.h != nullptr) {
      tma::store_2d(&maps.h, v0, (c * a.HV + hv) * DK, smem + S::o_sb + buf * S::sb_bytes);
      tma::store_commit();
    }

    // v_new = U - W S   (rows rg*16.., columns cg*32..)
    float acc[4][4];
    zero_acc<4>(acc);
    warp_mma_swz<4, DK / 16, AMajor::Row, BMajor::KN>(acc, w_tile, BT, rg * 16, 0, sb_tile, DK, cg * 32, 0, lane);
    const float glast = gs[BT - 1];
    {
      const int r_lo = rg * 16 + g, r_hi = r_lo + 8;
      const float e_lo = r_lo < cm.len ? exp2f(glast - gs[r_lo]) : 0.f;   // rows past the chunk's end contribute nothing
      const float e_hi = r_hi < cm.len ? exp2f(glast - gs[r_hi]) : 0.f;
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
        const int col = cg * 32 + nt * 8 + 2 * t;
        float2 u_lo = make_float2(0.f, 0.f), u_hi = make_float2(0.f, 0.f);
        if (has_u) {
          u_lo = unpack_bf16(lds32(swz_pair_addr(u_tile, BT, r_lo, col)));
          u_hi = unpack_bf16(lds32(swz_pair_addr(u_tile, BT, r_hi, col)));
        }
        const float v00 = u_lo.x - acc[nt][0], v01 = u_lo.y - acc[nt][1];
        const float v10 = u_hi.x - acc[nt][2], v11 = u_hi.y - acc[nt][3];
        sts32(swz_pair_addr(vn_tile, BT, r_lo, col), pack_bf16(v00, v01));
        sts32(swz_pair_addr(vn_tile, BT, r_hi, col), pack_bf16(v10, v11));
        sts32(swz_pair_addr(vt_tile, BT, r_lo, col), pack_bf16(v00 * e_lo, v01 * e_lo));
        sts32(swz_pair_addr(vt_tile, BT, r_hi, col), pack_bf16(v10 * e_hi, v11 * e_hi));
      }
    }
    tc5::fence_async_smem();
    if (tid == 0) {   // every store older than this step's h_c has released its shared tile
      if (a.h != nullptr) tma::store_wait_read<1>(); else tma::store_wait_read<0>();
    }
    bar_compute(2);
    if (a.v_new != nullptr) {
      if (cm.len == BT) {
        if (tid == 0) {
          tma::store_2d(&maps.vn, hv * DV + v0, cm.row, smem + S::o_vn + buf * S::u_bytes);
          tma::store_commit();
        }
      } else {
        __nv_bfloat16* vg = reinterpret_cast<__nv_bfloat16*>(a.v_new) + ((int64_t)cm.row * a.HV + hv) * DV + v0;
        for (int idx = tid; idx < BT * 8; idx += NCOMPUTE) {
          const int r = idx >> 3, ch = idx & 7;
          if (r < cm.len) {
            uint4 val;
            const uint32_t addr = swz_chunk_addr(vn_tile, BT, r, ch * 8);
            asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];\n" : "=r"(val.x), "=r"(val.y), "=r"(val.z), "=r"(val.w) : "r"(addr));
            *reinterpret_cast<uint4*>(vg + (int64_t)r * a.HV * DV + ch * 8) = val;
          }
        }
      }
    }

    // S <- 2^gamma_last S + K^T v~     (rows rg*(DK/4) + mt*16.., columns cg*32..)
    const float dec = exp2f(glast);
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
      for (int nt = 0; nt < 4; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) S_[mt][nt][e] *= dec;
      warp_mma_swz<4, BT / 16, AMajor::Trans, BMajor::KN>(S_[mt], k_tile, BT, rg * (DK / 4) + mt * 16, 0, vt_tile, BT, cg * 32,
                                                          0, lane);
    }
    __syncwarp();
    if (lane == 0) tc5::mbar_arrive(&empty[s]);   // this warp is done with stage s
    if (failed) break;
  }
  if (failed && lane == 0) atomicExch(&g_scan_fwd_timeout, 1);

  if (a.ht != nullptr) {
    float* ht = a.ht + ((int64_t)n * a.HV + hv) * DK * DV;
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
        int r = rg * (DK / 4) + mt * 16 + g;
        int col = v0 + cg * 32 + nt * 8 + 2 * t;
        *reinterpret_cast<float2*>(&ht[(int64_t)r * DV + col]) = make_float2(S_[mt][nt][0], S_[mt][nt][1]);
        *reinterpret_cast<float2*>(&ht[(int64_t)(r + 8) * DV + col]) = make_float2(S_[mt][nt][2], S_[mt][nt][3]);
      }
  }
  if (tid == 0) tma::store_wait_all<0>();   // shared tiles must outlive the stores that read them
}

template <int DK, int DV, int NSTAGE>
int launch(const b200gdn_chunk_args& a, cudaStream_t st) {
  using S = ScanFwdSmem<DK, NSTAGE>;
  static_assert(DV % BV == 0, "value dimension is processed in 64-column slices");
  if (int e = ensure_smem(scan_fwd_kernel<DK, DV, NSTAGE>, S::bytes)) return e;
  ScanFwdMaps m;
  const uint64_t pk = (uint64_t)a.H * DK, pw = (uint64_t)a.HV * DK, pv = (uint64_t)a.HV * DV;
  int rc = 0;
  rc |= tma::encode_bf16_2d(&m.w, a.w, a.rows, pw, pw, BT);
  rc |= tma::encode_bf16_2d(&m.k, a.k, a.rows, pk, pk, BT);
  // an absent tensor gets a well-formed map over k; it is never used
  if (a.u) rc |= tma::encode_bf16_2d(&m.u, a.u, a.rows, pv, pv, BT); else m.u = m.k;
  if (a.h) rc |= tma::encode_bf16_2d(&m.h, a.h, (uint64_t)a.n_chunks * a.HV * DK, DV, DV, DK); else m.h = m.k;
  if (a.v_new) rc |= tma::encode_bf16_2d(&m.vn, a.v_new, a.rows, pv, pv, BT); else m.vn = m.k;
  if (rc != 0) return set_error(B200GDN_ERR_CUDA, "scan_fwd: cuTensorMapEncodeTiled failed (%d)", rc);
  dim3 grid(DV / BV, a.HV, a.n_seq);
  scan_fwd_kernel<DK, DV, NSTAGE><<<grid, NTHREADS, S::bytes, st>>>(a, m);
  return check_launch("scan_fwd");
}

}  // namespace

int launch_scan_fwd(const b200gdn_chunk_args& a, cudaStream_t st) {
  if (a.K == 128 && a.V == 128) return launch<128, 128, 3>(a, st);
  if (a.K == 64 && a.V == 64) return launch<64, 64, 3>(a, st);
  return set_error(B200GDN_ERR_UNSUPPORTED, "scan_fwd: K=%d V=%d not built (64/64 and 128/128 are)", a.K, a.V);
}

}  // namespace gdn
