// Forward state scan: for every (sequence, value head) walk the chunks in order with the K x V fp32 state
// resident in tensor memory (TMEM):
//     h_c = S (bf16 snapshot, state at chunk start);  v_new = U - W S;
//     S <- 2^gamma_last S + (K 2^(gamma_last - gamma))^T v_new.
// Replaces chunk_gated_delta_rule_fwd_kernel_h_blockdim64 (fla/ops/common/chunk_delta_h.py:58-348).
//
// The recurrence is a chain of 64-row steps, so what matters is the latency of one step.  One CTA owns a
// 64-column slice of one state and is specialised by warp:
//   * producer warp: TMA (cp.async.bulk.tensor, 128-byte swizzle) fills a ring of NSTAGE stages with
//     W [64 x K], K [64 x K] and the U slice [64 x 64] of the chunks ahead; full/empty mbarriers;
//   * MMA warp (one thread): tcgen05.mma  V_acc = W S_bf16  (64 x 64 x K) and  S += K^T V~  (K x 64 x 64),
//     operands straight from the swizzled tiles, accumulators in TMEM; it also issues the TMA stores of
//     the state snapshot h_c and of v_new from double-buffered shared tiles;
//   * eight epilogue warps: read S from TMEM, round it to bf16 into shared memory, write it back scaled
//     by 2^gamma_last (tcgen05.st), and turn V_acc into v_new and the gated V~.
// Per step the chain is  S -> bf16 -> MMA -> v_new -> MMA, with four mbarrier hand-offs.
// A ragged last chunk is loaded as a full box (rows of the next sequence or zero fill); its extra rows
// are masked where v_new is formed, and its v_new rows are written with plain predicated stores.
//
// The same kernel produces the transition matrix of a whole shard for context parallelism
// (fla/ops/cp/chunk_delta_h.py:254-315): with u == NULL (zeros), h0 = identity and V := K the final
// state is M = prod_c (2^gamma_last I - K~^T W).
#include "tc5_tile.cuh"
#include "tma.cuh"

namespace gdn {
namespace {

constexpr int BV = 64;          // state columns per CTA
constexpr int NEPI = 256;       // 8 epilogue warps
constexpr int WARP_PROD = NEPI / 32, WARP_MMA = NEPI / 32 + 1;
constexpr int NTHREADS = NEPI + 64;
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
  static constexpr size_t bytes = o_bar + (2 * NSTAGE + 4) * 8 + 16 + 1024;  // + alignment slack
};

struct ScanFwdMaps {
  CUtensorMap w, k, u, h, vn;
};

template <int DK, int DV, int NSTAGE>
__global__ void __launch_bounds__(NTHREADS) scan_fwd_kernel(const b200gdn_chunk_args a, const __grid_constant__ ScanFwdMaps maps) {
  using S = ScanFwdSmem<DK, NSTAGE>;
  constexpr int NH = DK / 64;   // 16-row halves of the state per epilogue warp
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  float* gam_all = reinterpret_cast<float*>(smem + S::o_gam);
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + S::o_bar);
  uint64_t* empty = full + NSTAGE;
  uint64_t* s_ready = empty + NSTAGE;   // S accumulated (MMA 2 done)
  uint64_t* sb_ready = s_ready + 1;     // bf16 snapshot in shared memory, scaled S back in TMEM
  uint64_t* v_ready = sb_ready + 1;     // V_acc done (MMA 1)
  uint64_t* vt_ready = v_ready + 1;     // v_new / V~ tiles written
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(vt_ready + 1);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int v0 = blockIdx.x * BV, hv = blockIdx.y, n = blockIdx.z;
  const int G = a.HV / a.H, hq = hv / G;
  const int c_first = a.seq_meta[2 * n], nc = a.seq_meta[2 * n + 1];
  const bool has_u = a.u != nullptr;

  if (warp == 0) tc5::tmem_alloc(tmem_slot, 128);
  if (tid == 32) {
    for (int s = 0; s < NSTAGE; ++s) {
      tc5::mbar_init(&full[s], 1);    // producer's expect_tx arrive; the copies complete the transaction count
      tc5::mbar_init(&empty[s], 1);   // tcgen05.commit of the step's second MMA
    }
    tc5::mbar_init(s_ready, 1);
    tc5::mbar_init(sb_ready, NEPI / 32);
    tc5::mbar_init(v_ready, 1);
    tc5::mbar_init(vt_ready, NEPI / 32);
    tc5::fence_mbar_init();
  }
  tc5::fence_before_sync();
  __syncthreads();
  tc5::fence_after_sync();
  const uint32_t tm = *tmem_slot;
  const uint32_t TM_S = tm, TM_V = tm + 64;
  bool failed = false;

  if (warp == WARP_PROD) {
    // ================= producer warp: TMA loads =================
    if (lane == 0) {
      tma::prefetch_map(&maps.w);
      tma::prefetch_map(&maps.k);
      if (has_u) tma::prefetch_map(&maps.u);
    }
    const uint32_t tx_bytes = (uint32_t)(2 * S::w_bytes + (has_u ? S::u_bytes : 0) + BT * 4);
    if (lane == 0) {
      int row_next = nc > 0 ? load_chunk_meta(a.chunk_meta, c_first).row : 0;
      for (int ic = 0; ic < nc; ++ic) {
        const int s = ic % NSTAGE;
        const int row = row_next;
        if (ic + 1 < nc) row_next = load_chunk_meta(a.chunk_meta, c_first + ic + 1).row;   // one step ahead of its use
        if (ic >= NSTAGE && !tc5::mbar_wait(&empty[s], ((ic / NSTAGE) - 1) & 1)) { failed = true; break; }
        unsigned char* base = smem + (size_t)s * S::stage_bytes;
        tc5::mbar_expect_tx(&full[s], tx_bytes);
        tma::load_3d(base, &maps.w, row, (hv * DK) / 64, &full[s]);                 // W  [64 x K], all panels
        tma::load_3d(base + S::w_bytes, &maps.k, row, (hq * DK) / 64, &full[s]);    // K  [64 x K]
        if (has_u) tma::load_2d(base + 2 * S::w_bytes, &maps.u, hv * DV + v0, row, &full[s]);
        tma::load_1d(gam_all + s * BT, gamma_ptr(a.gamma, c_first + ic, a.HV, hv), BT * 4, &full[s]);
      }
    }
  } else if (warp == WARP_MMA) {
    // ================= MMA warp: one thread issues the contractions and the TMA stores =================
    if (lane == 0) {
      const uint32_t vt_addr = tc5::smem_addr(smem + S::o_vt);
      ChunkMeta cm_next = nc > 0 ? load_chunk_meta(a.chunk_meta, c_first) : ChunkMeta{0, 0, 0, 0};   // an empty sequence owns no chunk
      for (int ic = 0; ic < nc; ++ic) {
        const int c = c_first + ic, s = ic % NSTAGE, buf = ic & 1;
        const ChunkMeta cm = cm_next;
        if (ic + 1 < nc) cm_next = load_chunk_meta(a.chunk_meta, c + 1);
        const uint32_t w_addr = tc5::smem_addr(smem + (size_t)s * S::stage_bytes);
        const uint32_t k_addr = w_addr + (uint32_t)S::w_bytes;
        unsigned char* sb_ptr = smem + S::o_sb + buf * S::sb_bytes;
        if (!tc5::mbar_wait(&full[s], (ic / NSTAGE) & 1) || !tc5::mbar_wait(sb_ready, ic & 1)) { failed = true; break; }
        tc5::fence_after_sync();
        // V_acc = W S_bf16
        issue_mma_t<DK / 16>(TM_V, Operand{w_addr, BT, 0}, Operand{tc5::smem_addr(sb_ptr), DK, 1}, 64, BV, 0);
        tc5::mma_commit(v_ready);
        if (a.h != nullptr) {
          tma::store_2d(&maps.h, v0, (c * a.HV + hv) * DK, sb_ptr);
          tma::store_commit();
          // every store older than this h_c has released its shared tile before the next step re-writes it;
          // waiting here costs nothing, this thread would otherwise idle until the v_new tiles are ready
          tma::store_wait_read<1>();
        } else {
          tma::store_wait_read<0>();
        }
        if (!tc5::mbar_wait(vt_ready, ic & 1)) { failed = true; break; }
        tc5::fence_after_sync();
        // S += K^T V~
        issue_mma_t<BT / 16>(TM_S, Operand{k_addr, BT, 1}, Operand{vt_addr, BT, 1}, DK, BV, 1);
        tc5::mma_commit(s_ready);
        tc5::mma_commit(&empty[s]);
        if (a.v_new != nullptr && cm.len == BT) {
          tma::store_2d(&maps.vn, hv * DV + v0, cm.row, smem + S::o_vn + buf * S::u_bytes);
          tma::store_commit();
        }
      }
      tma::store_wait_all<0>();   // shared tiles must outlive the stores that read them
    }
  } else {
    // ================= epilogue warps =================
    const int q = warp & 3, hc = warp >> 2;
    const int g = lane >> 2, t = lane & 3;
    const uint32_t sb_base = smem_u32(smem + S::o_sb);
    const uint32_t vn_base = smem_u32(smem + S::o_vn);
    const uint32_t vt_tile = smem_u32(smem + S::o_vt);
    const int srow0 = (DK / 4) * q;           // first state row of this warp
    const uint32_t s_lane = (uint32_t)(32 * q) << 16;

    // state block of this thread: rows srow0 + 16*half + {g, g+8}, columns 32*hc + 8*i + 2t + {0,1}
    float Sr[NH][16];
    {
      const float* h0 = a.h0 ? a.h0 + ((int64_t)n * a.HV + hv) * DK * DV : nullptr;
#pragma unroll
      for (int hf = 0; hf < NH; ++hf)
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int r = srow0 + 16 * hf + g + ((e >> 1) << 3);
            const int col = v0 + 32 * hc + 8 * i + 2 * t + (e & 1);
            Sr[hf][4 * i + e] = h0 ? h0[(int64_t)r * DV + col] : 0.f;
          }
    }

    for (int ic = 0; ic < nc; ++ic) {
      const int c = c_first + ic, s = ic % NSTAGE, buf = ic & 1;
      const ChunkMeta cm = load_chunk_meta(a.chunk_meta, c);   // consumed late in the step
      const uint32_t u_tile = smem_u32(smem + (size_t)s * S::stage_bytes + 2 * S::w_bytes);
      const float* gs = gam_all + s * BT;
      const uint32_t sb_tile = sb_base + buf * (uint32_t)S::sb_bytes;
      const uint32_t vn_tile = vn_base + buf * (uint32_t)S::u_bytes;

      if (ic > 0) {
        if (!tc5::mbar_wait(s_ready, (ic - 1) & 1)) { failed = true; break; }
        tc5::fence_after_sync();
#pragma unroll
        for (int hf = 0; hf < NH; ++hf) tc5::tmem_ld_16x256b_x4(TM_S + s_lane + ((uint32_t)(16 * hf) << 16) + 32 * hc, Sr[hf]);
        tc5::tmem_ld_wait();
      }
      // bf16 snapshot (operand of W S and source of the h_c store) ...
#pragma unroll
      for (int hf = 0; hf < NH; ++hf) {
        FragStore fs;
#pragma unroll
        for (int i = 0; i < 4; ++i) fs.set(i, Sr[hf][4 * i], Sr[hf][4 * i + 1], Sr[hf][4 * i + 2], Sr[hf][4 * i + 3]);
        fs.store(sb_tile, DK, srow0 + 16 * hf, 32 * hc, lane);
      }
      // ... and the decayed state back to TMEM, where the second contraction accumulates onto it
      if (!tc5::mbar_wait(&full[s], (ic / NSTAGE) & 1)) { failed = true; break; }
      const float glast = gs[BT - 1];
      const float dec = fast_exp2(glast);
#pragma unroll
      for (int hf = 0; hf < NH; ++hf) {
#pragma unroll
        for (int e = 0; e < 16; ++e) Sr[hf][e] *= dec;
        tc5::tmem_st_16x256b_x4(TM_S + s_lane + ((uint32_t)(16 * hf) << 16) + 32 * hc, Sr[hf]);
      }
      tc5::tmem_st_wait();
      tc5::fence_async_smem();
      tc5::fence_before_sync();
      __syncwarp();
      if (lane == 0) tc5::mbar_arrive(sb_ready);

      // v_new = U - V_acc  (rows 16q + {g, g+8}, columns 32*hc ..)
      const int r_lo = 16 * q + g, r_hi = r_lo + 8;
      float2 u_lo[4], u_hi[4];
      {
        FragLoad fu;
        if (has_u) fu.load(u_tile, BT, 16 * q, 32 * hc, lane);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          u_lo[i] = has_u ? fu.lo2(i) : make_float2(0.f, 0.f);
          u_hi[i] = has_u ? fu.hi2(i) : make_float2(0.f, 0.f);
        }
      }
      // rows past the chunk's end contribute nothing: they are selected away (not multiplied by zero, their tiles may
      // hold anything, NaN bit patterns included)
      const bool ok_lo = r_lo < cm.len, ok_hi = r_hi < cm.len;
      const float e_lo = fast_exp2(glast - gs[r_lo]), e_hi = fast_exp2(glast - gs[r_hi]);
      if (!tc5::mbar_wait(v_ready, ic & 1)) { failed = true; break; }
      tc5::fence_after_sync();
      float acc[16];
      tc5::tmem_ld_16x256b_x4(TM_V + s_lane + 32 * hc, acc);
      tc5::tmem_ld_wait();
      FragStore fs_vn, fs_vt;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float v00 = ok_lo ? u_lo[i].x - acc[4 * i] : 0.f, v01 = ok_lo ? u_lo[i].y - acc[4 * i + 1] : 0.f;
        const float v10 = ok_hi ? u_hi[i].x - acc[4 * i + 2] : 0.f, v11 = ok_hi ? u_hi[i].y - acc[4 * i + 3] : 0.f;
        fs_vn.set(i, v00, v01, v10, v11);
        fs_vt.set(i, v00 * e_lo, v01 * e_lo, v10 * e_hi, v11 * e_hi);
      }
      fs_vn.store(vn_tile, BT, 16 * q, 32 * hc, lane);
      fs_vt.store(vt_tile, BT, 16 * q, 32 * hc, lane);
      tc5::fence_async_smem();
      tc5::fence_before_sync();
      __syncwarp();
      if (lane == 0) tc5::mbar_arrive(vt_ready);

      if (a.v_new != nullptr && cm.len < BT) {
        // ragged chunk: every warp writes the valid rows of its own block straight from its registers (no CTA-wide
        // barrier here: a warp whose bounded wait expired has left the loop and would never arrive at one)
        __nv_bfloat16* vg = reinterpret_cast<__nv_bfloat16*>(a.v_new) + ((int64_t)cm.row * a.HV + hv) * DV + v0 + 32 * hc + 2 * t;
        const int64_t vstride = (int64_t)a.HV * DV;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          if (r_lo < cm.len) *reinterpret_cast<uint32_t*>(vg + r_lo * vstride + 8 * i) = fs_vn.lo[i];
          if (r_hi < cm.len) *reinterpret_cast<uint32_t*>(vg + r_hi * vstride + 8 * i) = fs_vn.hi[i];
        }
      }
    }

    if (!failed && a.ht != nullptr) {
      if (nc > 0) {
        if (tc5::mbar_wait(s_ready, (nc - 1) & 1)) {
          tc5::fence_after_sync();
#pragma unroll
          for (int hf = 0; hf < NH; ++hf) tc5::tmem_ld_16x256b_x4(TM_S + s_lane + ((uint32_t)(16 * hf) << 16) + 32 * hc, Sr[hf]);
          tc5::tmem_ld_wait();
        } else {
          failed = true;
        }
      }
      float* ht = a.ht + ((int64_t)n * a.HV + hv) * DK * DV;
#pragma unroll
      for (int hf = 0; hf < NH; ++hf)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int r = srow0 + 16 * hf + g, col = v0 + 32 * hc + 8 * i + 2 * t;
          *reinterpret_cast<float2*>(&ht[(int64_t)r * DV + col]) = make_float2(Sr[hf][4 * i], Sr[hf][4 * i + 1]);
          *reinterpret_cast<float2*>(&ht[(int64_t)(r + 8) * DV + col]) = make_float2(Sr[hf][4 * i + 2], Sr[hf][4 * i + 3]);
        }
    }
  }

  if (failed && lane == 0) atomicExch(&g_scan_fwd_timeout, 1);
  tc5::fence_before_sync();
  __syncthreads();
  if (warp == 0) tc5::tmem_dealloc(tm, 128);
}

template <int DK, int DV, int NSTAGE>
int launch(const b200gdn_chunk_args& a, cudaStream_t st) {
  using S = ScanFwdSmem<DK, NSTAGE>;
  static_assert(DV % BV == 0, "value dimension is processed in 64-column slices");
  if (int e = ensure_smem(scan_fwd_kernel<DK, DV, NSTAGE>, S::bytes)) return e;
  ScanFwdMaps m;
  const uint64_t pk = (uint64_t)a.H * DK, pw = (uint64_t)a.HV * DK, pv = (uint64_t)a.HV * DV;
  int rc = 0;
  rc |= tma::encode_bf16_panels(&m.w, a.w, a.rows, pw, pw, BT, DK / 64);
  rc |= tma::encode_bf16_panels(&m.k, a.k, a.rows, pk, pk, BT, DK / 64);
  CUtensorMap dummy;
  rc |= tma::encode_bf16_2d(&dummy, a.k, a.rows, pk, pk, BT);
  // an absent tensor gets a well-formed map over k; it is never used
  if (a.u) rc |= tma::encode_bf16_2d(&m.u, a.u, a.rows, pv, pv, BT); else m.u = dummy;
  if (a.h) rc |= tma::encode_bf16_2d(&m.h, a.h, (uint64_t)a.n_chunks * a.HV * DK, DV, DV, DK); else m.h = dummy;
  if (a.v_new) rc |= tma::encode_bf16_2d(&m.vn, a.v_new, a.rows, pv, pv, BT); else m.vn = dummy;
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

// Reads and clears the flag a bounded device wait raises when it expires (synchronises with the device).
int scan_fwd_timeout_flag() {
  int v = 0, zero = 0;
  cudaMemcpyFromSymbol(&v, g_scan_fwd_timeout, sizeof(int));
  if (v) cudaMemcpyToSymbol(g_scan_fwd_timeout, &zero, sizeof(int));
  return v;
}

}  // namespace gdn
