// Reverse state-gradient scan: for every (sequence, value head) walk the chunks backwards with the K x V
// fp32 gradient dS resident in tensor memory (TMEM):
//     dh_c = dS (bf16 snapshot, gradient w.r.t. the state at chunk END)
//     dv2  = (K dS) 2^(gamma_last - gamma) + dv_local
//     dS  <- 2^gamma_last dS + (Q)^T (do scale 2^gamma) - W^T dv2
// Replaces chunk_gated_delta_rule_bwd_kernel_dhu_blockdim64 (fla/ops/common/chunk_delta_h.py:369-683) and, in its
// DVL form, chunk_bwd_kernel_dv_local (fla/ops/common/chunk_o.py:465-540) as well:
//     dv_local[j] = sum_{i >= j} scale <k_j, q_i> 2^(gamma_i - gamma_j) do_i
// is formed in the same CTA from the Q, K and do tiles the scan holds anyway, so dv_local never touches HBM.
//
// Same organisation as the forward scan: one CTA per 64-column slice of one state; a producer thread feeds
// a ring of stages with TMA (Q, K, W tiles, the do slice, gamma; the qk tile with DVL, the dv_local slice without);
// one thread issues tcgen05.mma  acc = K dS_bf16  and  dS += Q^T do_s - W^T dv2  with accumulators in TMEM and the
// TMA stores of dh_c and dv2; eight epilogue warps move dS between TMEM and shared memory and form dv2.
// DVL: the MMA thread also issues  L = qk^T do  of the NEXT chunk right after a step's last product (it only needs
// loaded tiles and runs while the epilogue warps convert dS); qk = tril(Q K^T 2^(gamma_i-gamma_j)) comes ready-made
// from the forward pass; the epilogue warps add scale L where they form dv2.
// Rows of a ragged last chunk (the first step of the reverse walk) that lie past its end are zeroed in the do and qk
// tiles before the first product, and where dv2 and do_s are formed.
//
// With zero do and dv_local, identity end gradient and V := K the result is the backward transition matrix of a shard
// for context parallelism (fla/ops/cp/chunk_delta_h.py:478-744).  When cp_dM is given the grid grows by K / 64 such
// slices (either form), so that the shard's (dh_ext, dM) pair comes out of ONE launch.  Without DVL, d_o == NULL also
// means zero do and dv_local, and dv2 is then not stored.
#include "tc5_tile.cuh"
#include "tma.cuh"

namespace gdn {
namespace {

constexpr int BV = 64;
constexpr int NEPI = 256;
constexpr int WARP_PROD = NEPI / 32, WARP_MMA = NEPI / 32 + 1;
__device__ int g_scan_bwd_timeout = 0;

template <int DK, int NSTAGE, bool DVL>
struct ScanBwdSmem {
  static constexpr size_t t_bytes = BT * DK * 2;            // Q, K, W tiles
  static constexpr size_t s_bytes = BT * BV * 2;            // do slice; dv_local slice or (DVL) the qk tile
  static constexpr size_t stage_bytes = 3 * t_bytes + 2 * s_bytes;
  static constexpr size_t o_sb = NSTAGE * stage_bytes;      // 2 x dS snapshot [DK][64]
  static constexpr size_t sb_bytes = DK * BV * 2;
  static constexpr size_t o_d2 = o_sb + 2 * sb_bytes;       // 2 x dv2 slice [64][64]
  static constexpr size_t o_dos = o_d2 + 2 * s_bytes;       // do scale 2^gamma [64][64]
  static constexpr size_t o_gam = o_dos + s_bytes;
  static constexpr size_t o_bar = o_gam + NSTAGE * BT * 4;
  static constexpr size_t bytes = o_bar + (3 * NSTAGE + 5) * 8 + 16 + 1024;
};

struct ScanBwdMaps {
  CUtensorMap q, k, w, d_o, dv2, dh, pq;
};

template <int DK, int DV, int NSTAGE, bool DVL>
__global__ void __launch_bounds__(NEPI + 64)
    scan_bwd_kernel(const b200gdn_chunk_args a, const __grid_constant__ ScanBwdMaps maps) {
  using S = ScanBwdSmem<DK, NSTAGE, DVL>;
  constexpr int NH = DK / 64;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  float* gam_all = reinterpret_cast<float*>(smem + S::o_gam);
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + S::o_bar);   // K, do, gamma (+ qk | dv_local): what a step needs first
  uint64_t* full2 = full + NSTAGE;      // Q, W: operands of the step's last products
  uint64_t* empty = full2 + NSTAGE;
  uint64_t* s_ready = empty + NSTAGE;   // dS accumulated (last product of a step done)
  uint64_t* sb_ready = s_ready + 1;     // bf16 snapshot in shared memory
  uint64_t* v_ready = sb_ready + 1;     // acc = K dS done
  uint64_t* vt_ready = v_ready + 1;     // dv2 / do_s tiles written, decayed dS back in TMEM
  uint64_t* l_ready = vt_ready + 1;     // DVL: L = qk^T do done
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(l_ready + 1);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  // CTAs past the DV / 64 value slices (launched only when cp_dM is given) scan the backward transition matrix of the
  // sequence instead: zero do and dv_local, identity end gradient, V := K, nothing stored but the final "gradient" dM
  const bool m_mode = (int)blockIdx.x >= DV / BV;
  const bool dvl = DVL && !m_mode;
  const int v0 = (m_mode ? (int)blockIdx.x - DV / BV : (int)blockIdx.x) * BV, hv = blockIdx.y, n = blockIdx.z;
  const int G = a.HV / a.H, hq = hv / G;
  const int c_first = a.seq_meta[2 * n], nc = a.seq_meta[2 * n + 1];
  const int c_last = c_first + nc - 1;
  const bool has_do = !m_mode && (DVL || a.d_o != nullptr);
  const bool has_dl = !m_mode && !DVL && a.d_o != nullptr;   // a dv_local slice comes in through the dv2 buffer
  const bool store_d2 = a.dv2 != nullptr && (dvl || has_dl);
  const bool st_dh = !m_mode && a.dh != nullptr;
  float* const dh0_out = m_mode ? a.cp_dM : a.dh0;
  const bool vfirst = !m_mode && (a.options & B200GDN_STATE_V_FIRST);   // dht and dh0 stored [V][K]
  constexpr uint32_t TMEM_COLS = DVL ? 256 : 128;   // DVL: 192 used; the allocation is a power of two

  if (warp == 0) tc5::tmem_alloc(tmem_slot, TMEM_COLS);
  if (tid == 32) {
    for (int s = 0; s < NSTAGE; ++s) {
      tc5::mbar_init(&full[s], 1);
      tc5::mbar_init(&full2[s], 1);
      tc5::mbar_init(&empty[s], 1);
    }
    tc5::mbar_init(s_ready, 1);
    tc5::mbar_init(sb_ready, NEPI / 32);
    tc5::mbar_init(v_ready, 1);
    tc5::mbar_init(vt_ready, NEPI / 32);
    tc5::mbar_init(l_ready, 1);
    tc5::fence_mbar_init();
  }
  tc5::fence_before_sync();
  __syncthreads();
  tc5::fence_after_sync();
  const uint32_t tm = *tmem_slot;
  const uint32_t TM_S = tm, TM_V = tm + 64, TM_L = tm + 128;   // the last one only with DVL
  bool failed = false;

  if (warp == WARP_PROD) {
    // ================= producer: TMA loads, chunks in reverse order =================
    if (lane == 0) {
      tma::prefetch_map(&maps.q);
      tma::prefetch_map(&maps.k);
      tma::prefetch_map(&maps.w);
      const uint32_t tx1 = (uint32_t)(S::t_bytes + ((has_do ? 1 : 0) + ((has_dl || dvl) ? 1 : 0)) * S::s_bytes + BT * 4);
      const uint32_t tx2 = (uint32_t)((has_do ? 2 : 1) * S::t_bytes);
      int row_next = nc > 0 ? load_chunk_meta(a.chunk_meta, c_last).row : 0;
      for (int ic = 0; ic < nc; ++ic) {
        const int s = ic % NSTAGE, c = c_last - ic;
        const int row = row_next;
        if (ic + 1 < nc) row_next = load_chunk_meta(a.chunk_meta, c - 1).row;
        if (dvl && ic + NSTAGE < nc) {
          // the ring is short: pull the tiles of the chunk that will take this stage next into L2 now
          const int row_pf = load_chunk_meta(a.chunk_meta, c - NSTAGE).row;
          tma::prefetch_3d(&maps.k, row_pf, (hq * DK) / 64);
          tma::prefetch_2d(&maps.d_o, hv * DV + v0, row_pf);
          tma::prefetch_2d(&maps.pq, hv * BT, row_pf);
          tma::prefetch_3d(&maps.q, row_pf, (hq * DK) / 64);
          tma::prefetch_3d(&maps.w, row_pf, (hv * DK) / 64);
        }
        if (ic >= NSTAGE && !tc5::mbar_wait(&empty[s], ((ic / NSTAGE) - 1) & 1)) { failed = true; break; }
        unsigned char* base = smem + (size_t)s * S::stage_bytes;
        // in the order the step needs them, on two barriers: the first product does not wait for Q and W
        tc5::mbar_expect_tx(&full[s], tx1);
        tma::load_3d(base + S::t_bytes, &maps.k, row, (hq * DK) / 64, &full[s]);
        if (has_do) tma::load_2d(base + 3 * S::t_bytes, &maps.d_o, hv * DV + v0, row, &full[s]);
        if (has_dl) tma::load_2d(base + 3 * S::t_bytes + S::s_bytes, &maps.dv2, hv * DV + v0, row, &full[s]);
        if (dvl) tma::load_2d(base + 3 * S::t_bytes + S::s_bytes, &maps.pq, hv * BT, row, &full[s]);
        tma::load_1d(gam_all + s * BT, gamma_ptr(a.gamma, c, a.HV, hv), BT * 4, &full[s]);
        tc5::mbar_expect_tx(&full2[s], tx2);
        if (has_do) tma::load_3d(base, &maps.q, row, (hq * DK) / 64, &full2[s]);
        tma::load_3d(base + 2 * S::t_bytes, &maps.w, row, (hv * DK) / 64, &full2[s]);
      }
    }
  } else if (warp == WARP_MMA) {
    // ================= MMA thread =================
    if (lane == 0) {
      const uint32_t dos_addr = tc5::smem_addr(smem + S::o_dos);
      ChunkMeta cm_next = nc > 0 ? load_chunk_meta(a.chunk_meta, c_last) : ChunkMeta{0, 0, 0, 0};   // an empty sequence owns no chunk
      for (int ic = 0; ic < nc && !failed; ++ic) {
        const int c = c_last - ic, s = ic % NSTAGE, buf = ic & 1;
        const ChunkMeta cm = cm_next;
        if (ic + 1 < nc) cm_next = load_chunk_meta(a.chunk_meta, c - 1);
        const uint32_t q_addr = tc5::smem_addr(smem + (size_t)s * S::stage_bytes);
        const uint32_t k_addr = q_addr + (uint32_t)S::t_bytes, w_addr = q_addr + 2 * (uint32_t)S::t_bytes;
        const uint32_t do_addr = q_addr + 3 * (uint32_t)S::t_bytes, pq_addr = do_addr + (uint32_t)S::s_bytes;
        unsigned char* sb_ptr = smem + S::o_sb + buf * S::sb_bytes;
        unsigned char* d2_ptr = smem + S::o_d2 + buf * S::s_bytes;
        if (!tc5::mbar_wait(&full[s], (ic / NSTAGE) & 1) || !tc5::mbar_wait(sb_ready, ic & 1)) { failed = true; break; }
        tc5::fence_after_sync();
        // acc = K dS_bf16
        issue_mma_t<DK / 16>(TM_V, Operand{k_addr, BT, 0}, Operand{tc5::smem_addr(sb_ptr), DK, 1}, 64, BV, 0);
        tc5::mma_commit(v_ready);
        if (dvl && ic == 0) {
          // L = qk^T do of the first step (the tails of a ragged chunk's tiles were zeroed before sb_ready)
          issue_mma_t<BT / 16>(TM_L, Operand{pq_addr, BT, 1}, Operand{do_addr, BT, 1}, 64, BV, 0);
          tc5::mma_commit(l_ready);
        }
        if (st_dh) {
          tma::store_2d(&maps.dh, v0, (c * a.HV + hv) * DK, sb_ptr);
          tma::store_commit();
          tma::store_wait_read<1>();   // older stores have released their tiles (re-written next step)
        } else {
          tma::store_wait_read<0>();
        }
        if (!tc5::mbar_wait(&full2[s], (ic / NSTAGE) & 1) || !tc5::mbar_wait(vt_ready, ic & 1)) { failed = true; break; }
        tc5::fence_after_sync();
        // dS += Q^T do_s - W^T dv2
        if (has_do) issue_mma_t<BT / 16>(TM_S, Operand{q_addr, BT, 1}, Operand{dos_addr, BT, 1}, DK, BV, 1);
        issue_mma_t<BT / 16>(TM_S, Operand{w_addr, BT, 1}, Operand{tc5::smem_addr(d2_ptr), BT, 1}, DK, BV, 1, /*neg_a=*/1);
        tc5::mma_commit(s_ready);
        tc5::mma_commit(&empty[s]);   // every product that reads this stage's tiles has been issued before this commit
        if (store_d2 && cm.len == BT) {
          tma::store_2d(&maps.dv2, hv * DV + v0, cm.row, d2_ptr);
          tma::store_commit();
        }
        if (dvl && ic + 1 < nc) {
          // L = qk^T do of the next step: it needs loaded tiles only and runs while the epilogue warps convert dS.
          // Waiting for those tiles here costs nothing, the next product of the chain needs them as well.
          const int s2 = (ic + 1) % NSTAGE;
          if (!tc5::mbar_wait(&full[s2], ((ic + 1) / NSTAGE) & 1)) { failed = true; break; }
          tc5::fence_after_sync();
          const uint32_t do2 = tc5::smem_addr(smem + (size_t)s2 * S::stage_bytes) + 3 * (uint32_t)S::t_bytes;
          issue_mma_t<BT / 16>(TM_L, Operand{do2 + (uint32_t)S::s_bytes, BT, 1}, Operand{do2, BT, 1}, 64, BV, 0);
          tc5::mma_commit(l_ready);
        }
      }
      tma::store_wait_all<0>();
    }
  } else if (warp < WARP_PROD) {
    // ================= epilogue warps =================
    const int q = warp & 3, hc = warp >> 2;
    const int g = lane >> 2, t = lane & 3;
    const uint32_t sb_base = smem_u32(smem + S::o_sb);
    const uint32_t d2_base = smem_u32(smem + S::o_d2);
    const uint32_t dos_tile = smem_u32(smem + S::o_dos);
    const int srow0 = (DK / 4) * q;
    const uint32_t s_lane = (uint32_t)(32 * q) << 16;

    float Sr[NH][16];
    {
      const float* dht = (a.dht && !m_mode) ? a.dht + ((int64_t)n * a.HV + hv) * DK * DV : nullptr;
#pragma unroll
      for (int hf = 0; hf < NH; ++hf)
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int r = srow0 + 16 * hf + g + ((e >> 1) << 3);
            const int col = v0 + 32 * hc + 8 * i + 2 * t + (e & 1);
            Sr[hf][4 * i + e] = dht ? (vfirst ? dht[(int64_t)col * DK + r] : dht[(int64_t)r * DV + col]) : ((m_mode && r == col) ? 1.f : 0.f);
          }
    }

    for (int ic = 0; ic < nc; ++ic) {
      const int c = c_last - ic, s = ic % NSTAGE, buf = ic & 1;
      const ChunkMeta cm = load_chunk_meta(a.chunk_meta, c);
      const uint32_t stage0 = smem_u32(smem + (size_t)s * S::stage_bytes);
      const uint32_t do_tile = stage0 + 3 * (uint32_t)S::t_bytes, dl_tile = do_tile + (uint32_t)S::s_bytes;
      const float* gs = gam_all + s * BT;
      const uint32_t sb_tile = sb_base + buf * (uint32_t)S::sb_bytes;
      const uint32_t d2_tile = d2_base + buf * (uint32_t)S::s_bytes;

      if (ic > 0) {
        if (!tc5::mbar_wait(s_ready, (ic - 1) & 1)) { failed = true; break; }
        tc5::fence_after_sync();
#pragma unroll
        for (int hf = 0; hf < NH; ++hf) tc5::tmem_ld_16x256b_x4(TM_S + s_lane + ((uint32_t)(16 * hf) << 16) + 32 * hc, Sr[hf]);
        tc5::tmem_ld_wait();
      }
      // bf16 snapshot: all the first product waits for ...
#pragma unroll
      for (int hf = 0; hf < NH; ++hf) {
        FragStore fs;
#pragma unroll
        for (int i = 0; i < 4; ++i) fs.set(i, Sr[hf][4 * i], Sr[hf][4 * i + 1], Sr[hf][4 * i + 2], Sr[hf][4 * i + 3]);
        fs.store(sb_tile, DK, srow0 + 16 * hf, 32 * hc, lane);
      }
      if (dvl && ic == 0 && cm.len < BT) {
        // ragged chunk (only the first step of the reverse walk can be one): rows past its end in the do and qk tiles
        // belong to the next sequence and must not enter the contraction over rows of L = qk^T do
        if (!tc5::mbar_wait(&full[s], 0)) { failed = true; break; }
        zero_tail_rows<BT, BV>(smem + (size_t)s * S::stage_bytes + 3 * S::t_bytes, cm.len, tid, NEPI);
        zero_tail_rows<BT, BV>(smem + (size_t)s * S::stage_bytes + 3 * S::t_bytes + S::s_bytes, cm.len, tid, NEPI);
      }
      tc5::fence_async_smem();
      __syncwarp();
      if (lane == 0) tc5::mbar_arrive(sb_ready);
      // ... and, while that product runs, the decayed gradient back to TMEM (ordered before the accumulating products
      // by the vt_ready hand-off below)
      if (!tc5::mbar_wait(&full[s], (ic / NSTAGE) & 1)) { failed = true; break; }
      const float glast = gs[BT - 1];
      const float dec = fast_exp2(glast);
#pragma unroll
      for (int hf = 0; hf < NH; ++hf) {
#pragma unroll
        for (int e = 0; e < 16; ++e) Sr[hf][e] *= dec;
        tc5::tmem_st_16x256b_x4(TM_S + s_lane + ((uint32_t)(16 * hf) << 16) + 32 * hc, Sr[hf]);
      }

      // do_s = do scale 2^gamma (rows past the chunk's end zeroed) into its own tile; dv_local into registers
      const int r_lo = 16 * q + g, r_hi = r_lo + 8;
      const bool ok_lo = r_lo < cm.len, ok_hi = r_hi < cm.len;
      const float q_lo = a.scale * fast_exp2(gs[r_lo]), q_hi = a.scale * fast_exp2(gs[r_hi]);
      const float e_lo = fast_exp2(glast - gs[r_lo]), e_hi = fast_exp2(glast - gs[r_hi]);
      float2 l_lo[4], l_hi[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) l_lo[i] = l_hi[i] = make_float2(0.f, 0.f);
      {
        if (has_dl) {
          FragLoad fl;
          fl.load(dl_tile, BT, 16 * q, 32 * hc, lane);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            l_lo[i] = fl.lo2(i);
            l_hi[i] = fl.hi2(i);
          }
        }
        if (has_do) {
          FragLoad fd;
          fd.load(do_tile, BT, 16 * q, 32 * hc, lane);
          FragStore fs;
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float2 d_lo = fd.lo2(i), d_hi = fd.hi2(i);
            fs.set(i, ok_lo ? d_lo.x * q_lo : 0.f, ok_lo ? d_lo.y * q_lo : 0.f, ok_hi ? d_hi.x * q_hi : 0.f,
                   ok_hi ? d_hi.y * q_hi : 0.f);
          }
          fs.store(dos_tile, BT, 16 * q, 32 * hc, lane);
        }
      }
      tc5::tmem_st_wait();
      if (!tc5::mbar_wait(v_ready, ic & 1)) { failed = true; break; }
      if (dvl && !tc5::mbar_wait(l_ready, ic & 1)) { failed = true; break; }
      tc5::fence_after_sync();
      float acc[16];
      tc5::tmem_ld_16x256b_x4(TM_V + s_lane + 32 * hc, acc);
      if (dvl) {
        float lv[16];
        tc5::tmem_ld_16x256b_x4(TM_L + s_lane + 32 * hc, lv);
        tc5::tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 4; ++i) {   // the qk tile carries no scale
          l_lo[i] = make_float2(lv[4 * i] * a.scale, lv[4 * i + 1] * a.scale);
          l_hi[i] = make_float2(lv[4 * i + 2] * a.scale, lv[4 * i + 3] * a.scale);
        }
      } else {
        tc5::tmem_ld_wait();
      }
      FragStore fs_d2;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float v00 = ok_lo ? acc[4 * i] * e_lo + l_lo[i].x : 0.f, v01 = ok_lo ? acc[4 * i + 1] * e_lo + l_lo[i].y : 0.f;
        const float v10 = ok_hi ? acc[4 * i + 2] * e_hi + l_hi[i].x : 0.f, v11 = ok_hi ? acc[4 * i + 3] * e_hi + l_hi[i].y : 0.f;
        fs_d2.set(i, v00, v01, v10, v11);
      }
      fs_d2.store(d2_tile, BT, 16 * q, 32 * hc, lane);
      tc5::fence_async_smem();
      tc5::fence_before_sync();
      __syncwarp();
      if (lane == 0) tc5::mbar_arrive(vt_ready);

      if (store_d2 && cm.len < BT) {
        // ragged chunk: every warp writes the valid rows of its own block straight from its registers (no CTA-wide
        // barrier here: a warp whose bounded wait expired has left the loop and would never arrive at one)
        __nv_bfloat16* vg = reinterpret_cast<__nv_bfloat16*>(a.dv2) + ((int64_t)cm.row * a.HV + hv) * DV + v0 + 32 * hc + 2 * t;
        const int64_t vstride = (int64_t)a.HV * DV;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          if (r_lo < cm.len) *reinterpret_cast<uint32_t*>(vg + r_lo * vstride + 8 * i) = fs_d2.lo[i];
          if (r_hi < cm.len) *reinterpret_cast<uint32_t*>(vg + r_hi * vstride + 8 * i) = fs_d2.hi[i];
        }
      }
    }

    if (!failed && dh0_out != nullptr) {
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
      float* d0 = dh0_out + ((int64_t)n * a.HV + hv) * DK * DV;
#pragma unroll
      for (int hf = 0; hf < NH; ++hf)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int r = srow0 + 16 * hf + g, col = v0 + 32 * hc + 8 * i + 2 * t;
          if (vfirst) {   // [V][K]: once per sequence, so the strided scalar stores do not matter
            d0[(int64_t)col * DK + r] = Sr[hf][4 * i];
            d0[(int64_t)(col + 1) * DK + r] = Sr[hf][4 * i + 1];
            d0[(int64_t)col * DK + r + 8] = Sr[hf][4 * i + 2];
            d0[(int64_t)(col + 1) * DK + r + 8] = Sr[hf][4 * i + 3];
          } else {
            *reinterpret_cast<float2*>(&d0[(int64_t)r * DV + col]) = make_float2(Sr[hf][4 * i], Sr[hf][4 * i + 1]);
            *reinterpret_cast<float2*>(&d0[(int64_t)(r + 8) * DV + col]) = make_float2(Sr[hf][4 * i + 2], Sr[hf][4 * i + 3]);
          }
        }
    }
  }

  if (failed && lane == 0) atomicExch(&g_scan_bwd_timeout, 1);
  tc5::fence_before_sync();
  __syncthreads();
  if (warp == 0) tc5::tmem_dealloc(tm, TMEM_COLS);
}

template <int DK, int DV, int NSTAGE, bool DVL>
int launch(const b200gdn_chunk_args& a, cudaStream_t st) {
  using S = ScanBwdSmem<DK, NSTAGE, DVL>;
  static_assert(DV % BV == 0, "value dimension is processed in 64-column slices");
  static_assert(S::bytes <= 227 * 1024, "shared memory of one CTA");
  static_assert(DK == DV, "the transition-matrix slices reuse the value-slice code with V := K");
  if (int e = ensure_smem(scan_bwd_kernel<DK, DV, NSTAGE, DVL>, S::bytes)) return e;
  ScanBwdMaps m;
  const uint64_t pk = (uint64_t)a.H * DK, pw = (uint64_t)a.HV * DK, pv = (uint64_t)a.HV * DV;
  int rc = 0;
  rc |= tma::encode_bf16_panels(&m.q, a.q, a.rows, pk, pk, BT, DK / 64);
  rc |= tma::encode_bf16_panels(&m.k, a.k, a.rows, pk, pk, BT, DK / 64);
  rc |= tma::encode_bf16_panels(&m.w, a.w, a.rows, pw, pw, BT, DK / 64);
  CUtensorMap dummy;
  rc |= tma::encode_bf16_2d(&dummy, a.k, a.rows, pk, pk, BT);
  // an absent tensor gets a well-formed map over k; it is never used
  if (a.dv2) rc |= tma::encode_bf16_2d(&m.dv2, a.dv2, a.rows, pv, pv, BT); else m.dv2 = dummy;
  if (a.d_o) rc |= tma::encode_bf16_2d(&m.d_o, a.d_o, a.rows, pv, pv, BT); else m.d_o = dummy;
  if (a.dh) rc |= tma::encode_bf16_2d(&m.dh, a.dh, (uint64_t)a.n_chunks * a.HV * DK, DV, DV, DK); else m.dh = dummy;
  if (DVL) rc |= tma::encode_bf16_2d(&m.pq, a.qk, a.rows, (uint64_t)a.HV * BT, (uint64_t)a.HV * BT, BT); else m.pq = dummy;
  if (rc != 0) return set_error(B200GDN_ERR_CUDA, "scan_bwd: cuTensorMapEncodeTiled failed (%d)", rc);
  dim3 grid(DV / BV + (a.cp_dM != nullptr ? DK / BV : 0), a.HV, a.n_seq);
  scan_bwd_kernel<DK, DV, NSTAGE, DVL><<<grid, NEPI + 64, S::bytes, st>>>(a, m);
  return check_launch(DVL ? "scan_dvl_bwd" : "scan_bwd");
}

}  // namespace

int launch_scan_bwd(const b200gdn_chunk_args& a, cudaStream_t st) {
  if (a.d_o != nullptr && a.dv2 == nullptr)
    return set_error(B200GDN_ERR_BAD_ARGUMENT, "scan_bwd: dv2 (holding dv_local) is required when d_o is given");
  if (a.K == 128 && a.V == 128) return launch<128, 128, 2, false>(a, st);
  if (a.K == 64 && a.V == 64) return launch<64, 64, 3, false>(a, st);
  return set_error(B200GDN_ERR_UNSUPPORTED, "scan_bwd: K=%d V=%d not built (64/64 and 128/128 are)", a.K, a.V);
}

// The reverse scan with dv_local formed on chip (needs d_o and the forward pass's qk; dv2 is an output only and may be NULL).
int launch_scan_dvl_bwd(const b200gdn_chunk_args& a, cudaStream_t st) {
  if (a.d_o == nullptr || a.qk == nullptr) return set_error(B200GDN_ERR_BAD_ARGUMENT, "scan_dvl_bwd: d_o or qk is NULL");
  if (a.K == 128 && a.V == 128) return launch<128, 128, 2, true>(a, st);
  if (a.K == 64 && a.V == 64) return launch<64, 64, 3, true>(a, st);
  return set_error(B200GDN_ERR_UNSUPPORTED, "scan_dvl_bwd: K=%d V=%d not built (64/64 and 128/128 are)", a.K, a.V);
}

// Reads and clears the flag a bounded device wait raises when it expires (synchronises with the device).
int scan_bwd_timeout_flag() {
  int v = 0, zero = 0;
  cudaMemcpyFromSymbol(&v, g_scan_bwd_timeout, sizeof(int));
  if (v) cudaMemcpyToSymbol(g_scan_bwd_timeout, &zero, sizeof(int));
  return v;
}

}  // namespace gdn
