// Forward state scan: for every (sequence, value head) walk the chunks in order with the K x V fp32 state
// resident in tensor memory (TMEM):
//     h_c = S (bf16 snapshot, state at chunk start);  v_new = U - W S;
//     S <- 2^gamma_last S + (K 2^(gamma_last - gamma))^T v_new.
// Replaces chunk_gated_delta_rule_fwd_kernel_h_blockdim64 (fla/ops/common/chunk_delta_h.py:58-348) and, in its
// OUT form, chunk_fwd_kernel_o (fla/ops/common/chunk_o.py:56-153) as well:
//     o = scale [ (Q h_c) 2^gamma + tril(Q K^T 2^(gamma_i - gamma_j)) v_new ]
// is formed in the same CTA from the state snapshot, the K tile and the v_new tile that are on chip anyway, so
// neither h nor v_new is read back from HBM for the output (they are still written for the backward pass).
//
// The recurrence is a chain of 64-row steps, so what matters is the latency of one step.  One CTA owns a
// 64-column slice of one state and is specialised by warp:
//   * producer warp: TMA (cp.async.bulk.tensor, 128-byte swizzle) fills a ring of NSTAGE stages with
//     W [64 x K], K [64 x K], the U slice [64 x 64] (and Q [64 x K]) of the chunks ahead; full/empty mbarriers;
//     in the OUT form the tiles of the chunk that will take a stage next are pulled into L2 at the same time;
//   * MMA warp (one thread): tcgen05.mma  V_acc = W S_bf16  (64 x 64 x K) and  S += K^T V~  (K x 64 x 64),
//     operands straight from the swizzled tiles, accumulators in TMEM; it also issues the TMA stores of
//     the state snapshot h_c and of v_new from double-buffered shared tiles.  OUT: the two products of the output
//     are off the chain: O1 = Q S_bf16 goes behind the first product (it runs while the epilogue warps form v_new)
//     and O2 = P~ v_new behind the second (it runs while they convert S), with P~ = tril(Q K^T 2^(gamma_i-gamma_j))
//     loaded ready-made (the intra-chunk kernel emits it), so nothing of the output waits on the chain's warps;
//   * eight epilogue warps: read S from TMEM, round it to bf16 into shared memory, write it back scaled
//     by 2^gamma_last (tcgen05.st), and turn V_acc into v_new and the gated V~;
//   * OUT: four output warps (one per TMEM lane quadrant) read O1 and O2, form scale (O1 2^gamma_i + O2) and store
//     o (one TMA store per warp, 16 rows).
// Per step the chain is  S -> bf16 -> MMA -> v_new -> MMA, with four mbarrier hand-offs; everything of the output
// runs in the shadow of that chain.  A tcgen05.mma of these shapes (N = 64) occupies the tensor pipe for about 45
// cycles per 16-deep step whatever M is, so the chain's products cost ~550 cycles per chunk and the output's ~540.
// A ragged last chunk is loaded as a full box (rows of the next sequence or zero fill); its extra rows
// are selected away where v_new is formed, and its v_new / o rows are written with plain predicated stores.
//
// The same kernel (without OUT) produces the transition matrix of a whole shard for context parallelism
// (fla/ops/cp/chunk_delta_h.py:254-315): with zero u, identity start state and V := K the final state is
// M = prod_c (2^gamma_last I - K~^T W).  When cp_M is given the grid grows by K / 64 such slices, so that the
// shard's (h_ext, M) pair comes out of ONE launch, as the reference's pre-process kernel does with its
// (cdiv(V,64) + cdiv(K,64), HV) grid (chunk_delta_h.py:41-315).
#include "tc5_tile.cuh"
#include "tma.cuh"

namespace gdn {
namespace {

constexpr int BV = 64;          // state columns per CTA
constexpr int NEPI = 256;       // 8 epilogue warps
constexpr int WARP_PROD = NEPI / 32, WARP_MMA = NEPI / 32 + 1;
constexpr int NOUT = 4;         // output warps (OUT form): warps WARP_MMA + 1 ..
__device__ int g_scan_fwd_timeout = 0;

template <int DK, int NSTAGE, bool OUT>
struct ScanFwdSmem {
  static constexpr size_t w_bytes = BT * DK * 2;            // W tile, K tile, Q tile
  static constexpr size_t u_bytes = BT * BV * 2;            // U slice, P~ tile, v_new / o slices
  static constexpr size_t o_qt = 2 * w_bytes + u_bytes;     // Q inside a stage
  static constexpr size_t o_pq = o_qt + w_bytes;            // P~ inside a stage
  static constexpr size_t stage_bytes = OUT ? o_pq + u_bytes : o_qt;
  static constexpr size_t o_sb = NSTAGE * stage_bytes;      // 2 x state snapshot [DK][64]
  static constexpr size_t sb_bytes = DK * BV * 2;
  static constexpr size_t o_vn = o_sb + 2 * sb_bytes;       // 2 x v_new slice [64][64]
  static constexpr size_t o_vt = o_vn + 2 * u_bytes;        // gated v_new slice
  static constexpr size_t o_os = o_vt + u_bytes;            // OUT: 2 x o staging [64][64]
  static constexpr size_t o_gam = o_os + (OUT ? 2 * u_bytes : 0);  // NSTAGE x 64 floats
  static constexpr size_t o_bar = o_gam + NSTAGE * BT * 4;
  static constexpr size_t bytes = o_bar + (3 * NSTAGE + 8) * 8 + 16 + 1024;  // + alignment slack
};

struct ScanFwdMaps {
  CUtensorMap w, k, u, h, vn, q, o, pq;
};

template <int DK, int DV, int NSTAGE, bool OUT>
__global__ void __launch_bounds__(NEPI + 64 + (OUT ? NOUT * 32 : 0))
    scan_fwd_kernel(const b200gdn_chunk_args a, const __grid_constant__ ScanFwdMaps maps) {
  using S = ScanFwdSmem<DK, NSTAGE, OUT>;
  constexpr int NH = DK / 64;   // 16-row halves of the state per epilogue warp
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  float* gam_all = reinterpret_cast<float*>(smem + S::o_gam);
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + S::o_bar);   // W, U, gamma of a stage (what the step needs first)
  uint64_t* full2 = full + NSTAGE;      // K (and Q, P~) of a stage
  uint64_t* empty = full2 + NSTAGE;
  uint64_t* s_ready = empty + NSTAGE;   // S accumulated (MMA 2 done)
  uint64_t* sb_ready = s_ready + 1;     // bf16 snapshot in shared memory
  uint64_t* v_ready = sb_ready + 1;     // V_acc done (MMA 1)
  uint64_t* vt_ready = v_ready + 1;     // v_new / V~ tiles written, decayed S back in TMEM
  // OUT, one pair of barriers per accumulator pair (chunk parity): a single barrier could complete two phases while a
  // slow output warp still waits for the first, and a parity wait cannot tell a phase from the one two later
  uint64_t* grp_ready = vt_ready + 1;   // [2] O1 and O2 of a chunk done
  uint64_t* o_free = grp_ready + 2;     // [2] the output warps have read the accumulator pair
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_free + 2);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  // CTAs past the DV / 64 value slices (launched only when cp_M is given) scan the transition matrix of the sequence
  // instead: zero u, identity start state, V := K, nothing stored but the final "state" M
  const bool m_mode = !OUT && (int)blockIdx.x >= DV / BV;
  const int v0 = (m_mode ? (int)blockIdx.x - DV / BV : (int)blockIdx.x) * BV, hv = blockIdx.y, n = blockIdx.z;
  const int G = a.HV / a.H, hq = hv / G;
  const int c_first = a.seq_meta[2 * n], nc = a.seq_meta[2 * n + 1];
  const bool has_u = !m_mode && a.u != nullptr;
  const bool st_h = !m_mode && a.h != nullptr, st_vn = !m_mode && a.v_new != nullptr;
  float* const ht_out = m_mode ? a.cp_M : a.ht;
  const bool vfirst = !m_mode && (a.options & B200GDN_STATE_V_FIRST);   // h0 and ht stored [V][K]
  constexpr uint32_t TMEM_COLS = OUT ? 512 : 128;   // 384 used; the allocation is a power of two

  if (warp == 0) tc5::tmem_alloc(tmem_slot, TMEM_COLS);
  if (tid == 32) {
    for (int s = 0; s < NSTAGE; ++s) {
      tc5::mbar_init(&full[s], 1);    // producer's expect_tx arrive; the copies complete the transaction count
      tc5::mbar_init(&full2[s], 1);
      // tcgen05.commit of the step's last MMA (+ OUT: the output warps are done with the stage's gate vector)
      tc5::mbar_init(&empty[s], OUT ? 1 + NOUT : 1);
    }
    tc5::mbar_init(s_ready, 1);
    tc5::mbar_init(sb_ready, NEPI / 32);
    tc5::mbar_init(v_ready, 1);
    tc5::mbar_init(vt_ready, NEPI / 32);
    tc5::mbar_init(&grp_ready[0], 1);
    tc5::mbar_init(&grp_ready[1], 1);
    tc5::mbar_init(&o_free[0], NOUT);
    tc5::mbar_init(&o_free[1], NOUT);
    tc5::fence_mbar_init();
  }
  tc5::fence_before_sync();
  __syncthreads();
  tc5::fence_after_sync();
  const uint32_t tm = *tmem_slot;
  // columns: S | V_acc | O1 x2 | O2 x2  (the last four only in the OUT form)
  const uint32_t TM_S = tm, TM_V = tm + 64, TM_O1 = tm + 128, TM_O2 = tm + 256;
  bool failed = false;

  if (warp == WARP_PROD) {
    // ================= producer warp: TMA loads =================
    if (lane == 0) {
      tma::prefetch_map(&maps.w);
      tma::prefetch_map(&maps.k);
      if (has_u) tma::prefetch_map(&maps.u);
      if (OUT) tma::prefetch_map(&maps.q);
    }
    const uint32_t tx1 = (uint32_t)(S::w_bytes + (has_u ? S::u_bytes : 0) + BT * 4);
    const uint32_t tx2 = (uint32_t)(S::w_bytes + (OUT ? S::w_bytes + S::u_bytes : 0));
    if (lane == 0) {
      int row_next = nc > 0 ? load_chunk_meta(a.chunk_meta, c_first).row : 0;
      for (int ic = 0; ic < nc; ++ic) {
        const int s = ic % NSTAGE;
        const int row = row_next;
        if (ic + 1 < nc) row_next = load_chunk_meta(a.chunk_meta, c_first + ic + 1).row;   // one step ahead of its use
        if (OUT && ic + NSTAGE < nc) {
          // the ring is short: pull the tiles of the chunk that will take this stage next into L2 now, so that its
          // copies see L2 latency when the stage is free again
          const int row_pf = load_chunk_meta(a.chunk_meta, c_first + ic + NSTAGE).row;
          tma::prefetch_3d(&maps.w, row_pf, (hv * DK) / 64);
          if (has_u) tma::prefetch_2d(&maps.u, hv * DV + v0, row_pf);
          tma::prefetch_3d(&maps.q, row_pf, (hq * DK) / 64);
          tma::prefetch_3d(&maps.k, row_pf, (hq * DK) / 64);
          tma::prefetch_2d(&maps.pq, hv * BT, row_pf);
        }
        if (ic >= NSTAGE && !tc5::mbar_wait(&empty[s], ((ic / NSTAGE) - 1) & 1)) { failed = true; break; }
        unsigned char* base = smem + (size_t)s * S::stage_bytes;
        // in the order the step needs them, on two barriers: the first product does not wait for K, Q and P~
        tc5::mbar_expect_tx(&full[s], tx1);
        tma::load_3d(base, &maps.w, row, (hv * DK) / 64, &full[s]);                 // W  [64 x K], all panels
        if (has_u) tma::load_2d(base + 2 * S::w_bytes, &maps.u, hv * DV + v0, row, &full[s]);
        tma::load_1d(gam_all + s * BT, gamma_ptr(a.gamma, c_first + ic, a.HV, hv), BT * 4, &full[s]);
        tc5::mbar_expect_tx(&full2[s], tx2);
        if (OUT) tma::load_3d(base + S::o_qt, &maps.q, row, (hq * DK) / 64, &full2[s]);   // Q  [64 x K]
        tma::load_3d(base + S::w_bytes, &maps.k, row, (hq * DK) / 64, &full2[s]);    // K  [64 x K]
        if (OUT) tma::load_2d(base + S::o_pq, &maps.pq, hv * BT, row, &full2[s]);    // P~ [64 x 64]
      }
    }
  } else if (warp == WARP_MMA) {
    // ================= MMA warp: one thread issues the contractions and the TMA stores =================
    if (lane == 0) {
      const uint32_t vt_addr = tc5::smem_addr(smem + S::o_vt);
      const uint32_t vn_addr0 = tc5::smem_addr(smem + S::o_vn);
      ChunkMeta cm_next = nc > 0 ? load_chunk_meta(a.chunk_meta, c_first) : ChunkMeta{0, 0, 0, 0};   // an empty sequence owns no chunk
      for (int ic = 0; ic < nc; ++ic) {
        const int c = c_first + ic, s = ic % NSTAGE, buf = ic & 1;
        const ChunkMeta cm = cm_next;
        if (ic + 1 < nc) cm_next = load_chunk_meta(a.chunk_meta, c + 1);
        const uint32_t w_addr = tc5::smem_addr(smem + (size_t)s * S::stage_bytes);
        const uint32_t k_addr = w_addr + (uint32_t)S::w_bytes, q_addr = w_addr + (uint32_t)S::o_qt;
        const uint32_t pq_addr = w_addr + (uint32_t)S::o_pq;
        unsigned char* sb_ptr = smem + S::o_sb + buf * S::sb_bytes;
        if (!tc5::mbar_wait(&full[s], (ic / NSTAGE) & 1) || !tc5::mbar_wait(sb_ready, ic & 1)) { failed = true; break; }
        tc5::fence_after_sync();
        // V_acc = W S_bf16
        issue_mma_t<DK / 16>(TM_V, Operand{w_addr, BT, 0}, Operand{tc5::smem_addr(sb_ptr), DK, 1}, 64, BV, 0);
        tc5::mma_commit(v_ready);
        if (!tc5::mbar_wait(&full2[s], (ic / NSTAGE) & 1)) { failed = true; break; }
        if (OUT) {
          // O1 = Q S_bf16, behind the first product: it runs while the epilogue warps form v_new.  The accumulator pair
          // of this parity was last used two chunks ago; the output warps have read it.
          if (ic >= 2 && !tc5::mbar_wait(&o_free[buf], ((ic >> 1) - 1) & 1)) { failed = true; break; }
          tc5::fence_after_sync();
          issue_mma_t<DK / 16>(TM_O1 + 64 * buf, Operand{q_addr, BT, 0}, Operand{tc5::smem_addr(sb_ptr), DK, 1}, 64, BV, 0);
        }
        if (st_h) {
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
        if (OUT) {
          // O2 = P~ v_new, behind the second product: it runs while the epilogue warps convert S
          issue_mma_t<BT / 16>(TM_O2 + 64 * buf, Operand{pq_addr, BT, 0}, Operand{vn_addr0 + buf * (uint32_t)S::u_bytes, BT, 1}, 64, BV, 0);
          tc5::mma_commit(&grp_ready[buf]);
        }
        tc5::mma_commit(&empty[s]);   // every product that reads this stage's tiles has been issued before this commit
        if (st_vn && cm.len == BT) {
          tma::store_2d(&maps.vn, hv * DV + v0, cm.row, smem + S::o_vn + buf * S::u_bytes);
          tma::store_commit();
        }
      }
      tma::store_wait_all<0>();   // shared tiles must outlive the stores that read them
    }
  } else if (warp < WARP_PROD) {
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
      const float* h0 = (a.h0 && !m_mode) ? a.h0 + ((int64_t)n * a.HV + hv) * DK * DV : nullptr;
#pragma unroll
      for (int hf = 0; hf < NH; ++hf)
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int r = srow0 + 16 * hf + g + ((e >> 1) << 3);
            const int col = v0 + 32 * hc + 8 * i + 2 * t + (e & 1);
            Sr[hf][4 * i + e] = h0 ? (vfirst ? h0[(int64_t)col * DK + r] : h0[(int64_t)r * DV + col]) : ((m_mode && r == col) ? 1.f : 0.f);
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
      // bf16 snapshot (operand of W S and source of the h_c store): all the first product waits for ...
#pragma unroll
      for (int hf = 0; hf < NH; ++hf) {
        FragStore fs;
#pragma unroll
        for (int i = 0; i < 4; ++i) fs.set(i, Sr[hf][4 * i], Sr[hf][4 * i + 1], Sr[hf][4 * i + 2], Sr[hf][4 * i + 3]);
        fs.store(sb_tile, DK, srow0 + 16 * hf, 32 * hc, lane);
      }
      tc5::fence_async_smem();
      __syncwarp();
      if (lane == 0) tc5::mbar_arrive(sb_ready);
      // ... and, while that product runs, the decayed state back to TMEM, where the second contraction accumulates
      // onto it (ordered before that contraction by the vt_ready hand-off below)
      if (!tc5::mbar_wait(&full[s], (ic / NSTAGE) & 1)) { failed = true; break; }
      const float glast = gs[BT - 1];
      const float dec = fast_exp2(glast);
#pragma unroll
      for (int hf = 0; hf < NH; ++hf) {
#pragma unroll
        for (int e = 0; e < 16; ++e) Sr[hf][e] *= dec;
        tc5::tmem_st_16x256b_x4(TM_S + s_lane + ((uint32_t)(16 * hf) << 16) + 32 * hc, Sr[hf]);
      }

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
      tc5::tmem_st_wait();
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

      if (st_vn && cm.len < BT) {
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

    if (!failed && ht_out != nullptr) {
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
      float* ht = ht_out + ((int64_t)n * a.HV + hv) * DK * DV;
#pragma unroll
      for (int hf = 0; hf < NH; ++hf)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int r = srow0 + 16 * hf + g, col = v0 + 32 * hc + 8 * i + 2 * t;
          if (vfirst) {   // [V][K]: once per sequence, so the strided scalar stores do not matter
            ht[(int64_t)col * DK + r] = Sr[hf][4 * i];
            ht[(int64_t)(col + 1) * DK + r] = Sr[hf][4 * i + 1];
            ht[(int64_t)col * DK + r + 8] = Sr[hf][4 * i + 2];
            ht[(int64_t)(col + 1) * DK + r + 8] = Sr[hf][4 * i + 3];
          } else {
            *reinterpret_cast<float2*>(&ht[(int64_t)r * DV + col]) = make_float2(Sr[hf][4 * i], Sr[hf][4 * i + 1]);
            *reinterpret_cast<float2*>(&ht[(int64_t)(r + 8) * DV + col]) = make_float2(Sr[hf][4 * i + 2], Sr[hf][4 * i + 3]);
          }
        }
    }
  } else if (OUT) {
    // ================= output warps: one per TMEM lane quadrant, rows 16 qd .. 16 qd + 15 of the chunk =================
    const int qd = warp & 3;
    const int g = lane >> 2, t = lane & 3;
    const int r_lo = 16 * qd + g, r_hi = r_lo + 8;
    const uint32_t lane_off = (uint32_t)(32 * qd) << 16;
    const uint32_t os_base = smem_u32(smem + S::o_os);
    for (int j = 0; j < nc; ++j) {
      const int s = j % NSTAGE, buf = j & 1;
      const ChunkMeta cm = load_chunk_meta(a.chunk_meta, c_first + j);
      if (!tc5::mbar_wait(&grp_ready[buf], (j >> 1) & 1)) { failed = true; break; }
      tc5::fence_after_sync();
      // o = scale (O1 2^gamma_i + O2)
      float o1[2][16], o2[2][16];
      tc5::tmem_ld_16x256b_x4(TM_O1 + 64 * buf + lane_off, o1[0]);
      tc5::tmem_ld_16x256b_x4(TM_O1 + 64 * buf + lane_off + 32, o1[1]);
      tc5::tmem_ld_16x256b_x4(TM_O2 + 64 * buf + lane_off, o2[0]);
      tc5::tmem_ld_16x256b_x4(TM_O2 + 64 * buf + lane_off + 32, o2[1]);
      const float* gs = gam_all + s * BT;
      const float e_lo = a.scale * fast_exp2(gs[r_lo]), e_hi = a.scale * fast_exp2(gs[r_hi]);
      tc5::tmem_ld_wait();
      tc5::fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        tc5::mbar_arrive(&o_free[buf]);   // the accumulator pair may be overwritten
        tc5::mbar_arrive(&empty[s]);      // the stage's gate vector is no longer needed here
      }
      FragStore fo[2];
#pragma unroll
      for (int b = 0; b < 2; ++b)
#pragma unroll
        for (int i = 0; i < 4; ++i)
          fo[b].set(i, o1[b][4 * i] * e_lo + o2[b][4 * i] * a.scale, o1[b][4 * i + 1] * e_lo + o2[b][4 * i + 1] * a.scale,
                    o1[b][4 * i + 2] * e_hi + o2[b][4 * i + 2] * a.scale, o1[b][4 * i + 3] * e_hi + o2[b][4 * i + 3] * a.scale);
      if (cm.len == BT) {
        const uint32_t os_tile = os_base + buf * (uint32_t)S::u_bytes;
        // this warp's own store of two chunks ago has finished reading the staging rows it is about to rewrite
        if (lane == 0) tma::store_wait_read<1>();
        __syncwarp();
        fo[0].store(os_tile, BT, 16 * qd, 0, lane);
        fo[1].store(os_tile, BT, 16 * qd, 32, lane);
        tc5::fence_async_smem();
        __syncwarp();
        if (lane == 0) {
          // 16 rows of the swizzled tile are 2 KiB on a 1 KiB boundary: a box of their own
          tma::store_2d(&maps.o, hv * DV + v0, cm.row + 16 * qd, smem + S::o_os + buf * S::u_bytes + (size_t)qd * 16 * 128);
          tma::store_commit();
        }
      } else {
        __nv_bfloat16* og = reinterpret_cast<__nv_bfloat16*>(a.o) + ((int64_t)cm.row * a.HV + hv) * DV + v0 + 2 * t;
        const int64_t ostride = (int64_t)a.HV * DV;
#pragma unroll
        for (int b = 0; b < 2; ++b)
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            if (r_lo < cm.len) *reinterpret_cast<uint32_t*>(og + r_lo * ostride + 32 * b + 8 * i) = fo[b].lo[i];
            if (r_hi < cm.len) *reinterpret_cast<uint32_t*>(og + r_hi * ostride + 32 * b + 8 * i) = fo[b].hi[i];
          }
      }
    }
    if (lane == 0) tma::store_wait_all<0>();   // the staging tiles must outlive the stores that read them
  }

  if (failed && lane == 0) atomicExch(&g_scan_fwd_timeout, 1);
  tc5::fence_before_sync();
  __syncthreads();
  if (warp == 0) tc5::tmem_dealloc(tm, TMEM_COLS);
}

template <int DK, int DV, int NSTAGE, bool OUT>
int launch(const b200gdn_chunk_args& a, cudaStream_t st) {
  using S = ScanFwdSmem<DK, NSTAGE, OUT>;
  static_assert(DV % BV == 0, "value dimension is processed in 64-column slices");
  static_assert(S::bytes <= 227 * 1024, "shared memory of one CTA");
  static_assert(DK == DV, "the transition-matrix slices reuse the value-slice code with V := K");
  if (int e = ensure_smem(scan_fwd_kernel<DK, DV, NSTAGE, OUT>, S::bytes)) return e;
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
  if (OUT) {
    rc |= tma::encode_bf16_panels(&m.q, a.q, a.rows, pk, pk, BT, DK / 64);
    rc |= tma::encode_bf16_2d(&m.o, a.o, a.rows, pv, pv, 16);   // one output warp stores 16 rows
    rc |= tma::encode_bf16_2d(&m.pq, a.qk, a.rows, (uint64_t)a.HV * BT, (uint64_t)a.HV * BT, BT);
  } else {
    m.q = dummy;
    m.o = dummy;
    m.pq = dummy;
  }
  if (rc != 0) return set_error(B200GDN_ERR_CUDA, "scan_fwd: cuTensorMapEncodeTiled failed (%d)", rc);
  dim3 grid(DV / BV + ((!OUT && a.cp_M != nullptr) ? DK / BV : 0), a.HV, a.n_seq);
  scan_fwd_kernel<DK, DV, NSTAGE, OUT><<<grid, NEPI + 64 + (OUT ? NOUT * 32 : 0), S::bytes, st>>>(a, m);
  return check_launch(OUT ? "scan_out_fwd" : "scan_fwd");
}

}  // namespace

int launch_scan_fwd(const b200gdn_chunk_args& a, cudaStream_t st) {
  if (a.K == 128 && a.V == 128) return launch<128, 128, 3, false>(a, st);
  if (a.K == 64 && a.V == 64) return launch<64, 64, 3, false>(a, st);
  return set_error(B200GDN_ERR_UNSUPPORTED, "scan_fwd: K=%d V=%d not built (64/64 and 128/128 are)", a.K, a.V);
}

// The scan and the chunk output in one kernel (needs q, qk and o in addition to the scan's arguments).
int launch_scan_out_fwd(const b200gdn_chunk_args& a, cudaStream_t st) {
  if (a.qk == nullptr) return set_error(B200GDN_ERR_BAD_ARGUMENT, "scan_out_fwd: qk (written by the intra stage) is NULL");
  if (a.K == 128 && a.V == 128) return launch<128, 128, 2, true>(a, st);
  if (a.K == 64 && a.V == 64) return launch<64, 64, 3, true>(a, st);
  return set_error(B200GDN_ERR_UNSUPPORTED, "scan_out_fwd: K=%d V=%d not built (64/64 and 128/128 are)", a.K, a.V);
}

// Reads and clears the flag a bounded device wait raises when it expires (synchronises with the device).
int scan_fwd_timeout_flag() {
  int v = 0, zero = 0;
  cudaMemcpyFromSymbol(&v, g_scan_fwd_timeout, sizeof(int));
  if (v) cudaMemcpyToSymbol(g_scan_fwd_timeout, &zero, sizeof(int));
  return v;
}

}  // namespace gdn
