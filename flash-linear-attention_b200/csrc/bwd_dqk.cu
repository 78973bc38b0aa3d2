// Chunk-local gradients of q and k and of the cumulative gate, on tcgen05 tensor cores with TMEM
// accumulators (replaces chunk_bwd_kernel_dqkwg of fla/ops/common/chunk_o.py:172-342 except for dw,
// which the WY-backward kernel forms itself so that it never touches HBM):
//     dP   = tril(do v_new^T 2^(gamma_i - gamma_j)) scale
//     dq   = (do scale 2^gamma) h^T + dP k
//     dk   = dP^T q + (v_new 2^(gamma_last - gamma)) dh^T
//     dG_i = <dq_i,q_i> - <dk_i,k_i>  (+ at the last valid row: 2^gamma_last <h,dh> + sum_i <dk_state_i,k_i>)
//
// One CTA of eight warps per (chunk, q/k head), looping over the value heads of the group.  All tiles
// arrive by TMA (one issuing thread) in the 128-byte-swizzled layout; one thread issues tcgen05.mma; the
// 64-row accumulators (dq | dk_state, dP, dk_intra) share 256 TMEM columns; the epilogues are spread over
// eight warps (warps w and w+4 share TMEM quadrant w&3 and split the columns).  h and dh are streamed in
// 64-column panels through one buffer pair, which keeps the CTA at ~106 KiB of shared memory, so two CTAs
// per SM overlap each other's phases.
#include "tc5_tile.cuh"
#include "tma.cuh"

namespace gdn {
namespace {

constexpr int NTHREADS = 256;
__device__ int g_dqk_timeout = 0;

template <int DK, int DV>
struct DqkSmem {
  static constexpr size_t o_do = 0;
  static constexpr size_t o_vn = o_do + BT * DV * 2;
  static constexpr size_t o_q = o_vn + BT * DV * 2;
  static constexpr size_t o_k = o_q + BT * DK * 2;
  static constexpr size_t o_hp = o_k + BT * DK * 2;      // h panel  [DK][64]; later output staging
  static constexpr size_t o_dhp = o_hp + DK * 128;       // dh panel [DK][64]
  static constexpr size_t o_p = o_dhp + DK * 128;        // dP~ [64][64]
  static constexpr size_t o_vec = o_p + BT * 128;
  static constexpr size_t bytes = o_vec + 2048 + 1024;   // + vectors + alignment slack
  static_assert(2 * DK * 128 >= BT * DK * 2, "staging fits in the panel buffers");
};

struct DqkMaps {
  CUtensorMap q, k, d_o, vn, h, dh, dk, dq;
};

// GROUPED: more than one value head per q/k head (their dq / dk contributions add up in fp32 through dq_acc and
// dk_part); the common ungrouped case is compiled without that path.
template <int DK, int DV, bool GROUPED>
__global__ void __launch_bounds__(NTHREADS, 2) bwd_dqk_kernel(const b200gdn_chunk_args a, const __grid_constant__ DqkMaps maps,
                                                              const int pf_dist) {
  using S = DqkSmem<DK, DV>;
  constexpr int NP = DV / 64;   // value panels
  constexpr int KB = DK / 64;   // 32-column blocks of a K-wide accumulator per warp
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* Do = smem + S::o_do;
  unsigned char* Vn = smem + S::o_vn;
  unsigned char* Qs = smem + S::o_q;
  unsigned char* Ks = smem + S::o_k;
  unsigned char* Hp = smem + S::o_hp;
  unsigned char* dHp = smem + S::o_dhp;
  unsigned char* Ps = smem + S::o_p;
  float* gs = reinterpret_cast<float*>(smem + S::o_vec);
  float* rqs = gs + BT;          // [2][64] row-dot partials <dq, q> of the two column halves
  float* rks = rqs + 2 * BT;     // [2][64] <dk, k>
  float* red = rks + 2 * BT;     // [0..7] <h,dh> per warp, [8..15] sum of <dk_state, k> per warp
  float* rq2s = red + 16;        // [2][64] <dq, q> of the group's summed dq (fused L2-norm backward, grouped heads only)
  uint64_t* bar = reinterpret_cast<uint64_t*>(rq2s + 2 * BT);
  uint64_t* bar_a = bar + 1;   // do, v_new, gamma of one head
  uint64_t* bar_b = bar + 2;   // one h / dh panel pair
  uint64_t* bar_c = bar + 3;   // q, k (once)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar + 4);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int q = warp & 3, hc = warp >> 2;
  const int g = lane >> 2, t = lane & 3;
  const int c = blockIdx.x, hq = blockIdx.y;
  const int G = GROUPED ? a.HV / a.H : 1;
  const ChunkMeta cm = load_chunk_meta(a.chunk_meta, c);
  const int64_t row0 = cm.row;
  const int r_lo = q * 16 + g, r_hi = r_lo + 8;
  const int cs = hc * 32, ck = hc * (DK / 2);

  // Loads of one head, in the order the phases need them, each group on its own barrier so that phase 1
  // starts as soon as do and v_new are in.  The second h / dh panel pair is only pulled into L2 here; it
  // takes the place of the first pair once phase 2 has consumed that.
  auto issue_loads = [&](int gi) {   // one thread
    const int hv = hq * G + gi;
    const int hrow = (c * a.HV + hv) * DK;
    tc5::mbar_expect_tx(bar_a, (uint32_t)(2 * BT * DV * 2 + BT * 4));
    tma::load_3d(Do, &maps.d_o, cm.row, (hv * DV) / 64, bar_a);
    tma::load_3d(Vn, &maps.vn, cm.row, (hv * DV) / 64, bar_a);
    tma::load_1d(gs, gamma_ptr(a.gamma, c, a.HV, hv), BT * 4, bar_a);
    tc5::mbar_expect_tx(bar_b, 2 * DK * 128);
    tma::load_2d(Hp, &maps.h, 0, hrow, bar_b);
    tma::load_2d(dHp, &maps.dh, 0, hrow, bar_b);
    if (gi == 0) {
      tc5::mbar_expect_tx(bar_c, 2 * BT * DK * 2);
      tma::load_3d(Qs, &maps.q, cm.row, (hq * DK) / 64, bar_c);
      tma::load_3d(Ks, &maps.k, cm.row, (hq * DK) / 64, bar_c);
    }
    for (int p = 1; p < NP; ++p) {
      tma::prefetch_2d(&maps.h, p * 64, hrow);
      tma::prefetch_2d(&maps.dh, p * 64, hrow);
    }
  };
  if (tid == 0) {
    tc5::mbar_init(bar, 1);
    tc5::mbar_init(bar_a, 1);
    tc5::mbar_init(bar_b, 1);
    tc5::mbar_init(bar_c, 1);
    tc5::fence_mbar_init();
    issue_loads(0);   // the first head's tiles are on their way while the CTA sets itself up
  }
  if (warp == 1) tc5::tmem_alloc(tmem_slot, 256);
  tc5::fence_before_sync();
  __syncthreads();
  tc5::fence_after_sync();
  const uint32_t tm = *tmem_slot;
  const uint32_t TM_DQ = tm, TM_DKS = tm + 128, TM_DP = tm + 128, TM_DKI = tm;
  PhaseBarrier ph{bar, 0u, &g_dqk_timeout};
  uint32_t par_b = 0;
  bool failed = false;

  const Operand opQ{tc5::smem_addr(Qs), BT, 1};   // B of dP~^T q : (k = token, n = key dim)
  const Operand opK{tc5::smem_addr(Ks), BT, 1};   // B of dP~ k
  const Operand opPk{tc5::smem_addr(Ps), BT, 0};  // dP~ as A(m = i, k = j)
  const Operand opPm{tc5::smem_addr(Ps), BT, 1};  // dP~ as A(m = j, k = i)

  for (int gi = 0; gi < G && !failed; ++gi) {
    const int hv = hq * G + gi;
    const bool first = gi == 0, last = gi == G - 1;
    const int hrow = (c * a.HV + hv) * DK;   // first row of this head's state snapshot in the [.., V] view
    if (gi > 0) {
      __syncthreads();  // previous head fully consumed (staging, gs, partials)
      if (tid == 0) issue_loads(gi);
    }
    if (first && tid == 32) {   // while everybody waits for the first tiles
      int c2, h2;
      // L2 look-ahead for the CTA that will follow this one: only what its first phase waits for (a look-ahead
      // over all of its tiles costs more in L2 evictions than it saves)
      if (successor_cta(pf_dist, c2, h2)) {
        const int row2 = load_chunk_meta(a.chunk_meta, c2).row, hv2 = h2 * G;
        tma::prefetch_3d(&maps.d_o, row2, (hv2 * DV) / 64);
        tma::prefetch_3d(&maps.vn, row2, (hv2 * DV) / 64);
        tma::prefetch_line(gamma_ptr(a.gamma, c2, a.HV, hv2));
        tma::prefetch_line(gamma_ptr(a.gamma, c2, a.HV, hv2) + 32);
      }
    }
    if (!tc5::mbar_wait(bar_a, gi & 1)) failed = true;
    if (cm.len < BT) {   // ragged chunk: the extra rows of the boxes belong to the next sequence
      zero_tail_rows<BT, DV>(Do, cm.len, tid, NTHREADS);
      zero_tail_rows<BT, DV>(Vn, cm.len, tid, NTHREADS);
      tc5::fence_async_smem();
    }
    if (__syncthreads_or(failed)) { failed = true; break; }

    // ---- phase 1: dP = do v_new^T
    if (tid == 0) {
      tc5::fence_after_sync();
      issue_mma_t<DV / 16>(TM_DP, Operand{tc5::smem_addr(Do), BT, 0}, Operand{tc5::smem_addr(Vn), BT, 0}, 64, 64, 0);
      ph.commit();
    }
    const float g_lo = gs[r_lo], g_hi = gs[r_hi], glast = gs[BT - 1];
    float hd = 0.f;  // <h, dh> partial of this thread
    auto add_hd = [&]() {
      for (int idx = tid; idx < DK * 8; idx += NTHREADS) {  // 16-byte chunks; same position in both panels
        uint4 x = *reinterpret_cast<const uint4*>(Hp + idx * 16);
        uint4 y = *reinterpret_cast<const uint4*>(dHp + idx * 16);
        const uint32_t* xu = reinterpret_cast<const uint32_t*>(&x);
        const uint32_t* yu = reinterpret_cast<const uint32_t*>(&y);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float2 p = unpack_bf16(xu[e]), q2 = unpack_bf16(yu[e]);
          hd += p.x * q2.x + p.y * q2.y;
        }
      }
    };
    if (!tc5::mbar_wait(bar_b, par_b)) failed = true;
    par_b ^= 1u;
    add_hd();
    if (first) {
      if (!tc5::mbar_wait(bar_c, 0)) failed = true;
      if (cm.len < BT) {
        zero_tail_rows<BT, DK>(Qs, cm.len, tid, NTHREADS);
        zero_tail_rows<BT, DK>(Ks, cm.len, tid, NTHREADS);
      }
    }
    if (__syncthreads_or(failed || !ph.wait())) { failed = true; break; }

    // ---- epilogue 1: dP~ -> shared; rescale the rows of do in place (v_new stays as loaded: its row factor
    //      2^(gamma_last - gamma_j) multiplies the rows of dk_state in the last epilogue instead)
    {
      float r[16];
      acc_ld32q(TM_DP, q, cs, r);
      tc5::tmem_ld_wait();
      FragStore fs;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int j0 = cs + i * 8 + 2 * t;
        float v[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int ii = (e & 2) ? r_hi : r_lo, jj = j0 + (e & 1);
          v[e] = (ii >= jj) ? r[4 * i + e] * a.scale * fast_exp2(((e & 2) ? g_hi : g_lo) - gs[jj]) : 0.f;
        }
        fs.set(i, v[0], v[1], v[2], v[3]);
      }
      fs.store(Ps, BT, q * 16, cs, lane);
    }
    for (int idx = tid; idx < BT * DV / 8; idx += NTHREADS) {
      const int row = (idx % (BT * 8)) / 8;
      const float fo = a.scale * fast_exp2(gs[row]);
      uint4* po = reinterpret_cast<uint4*>(Do + idx * 16);
      uint4 x = *po;
      uint32_t* xu = reinterpret_cast<uint32_t*>(&x);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float2 p = unpack_bf16(xu[e]);
        xu[e] = pack_bf16(p.x * fo, p.y * fo);
      }
      *po = x;
    }
    tc5::fence_async_smem();
    tc5::fence_before_sync();
    __syncthreads();

    // ---- phase 2: dq = do_s h^T + dP~ k ; dk_state = v_new dh^T (row factor later); h, dh streamed by 64-column panels
    for (int p = 0; p < NP && !failed; ++p) {
      if (p > 0) {
        if (tid == 0) {
          tc5::mbar_expect_tx(bar_b, 2 * DK * 128);
          tma::load_2d(Hp, &maps.h, p * 64, hrow, bar_b);
          tma::load_2d(dHp, &maps.dh, p * 64, hrow, bar_b);
        }
        if (!tc5::mbar_wait(bar_b, par_b)) failed = true;
        par_b ^= 1u;
        if (__syncthreads_or(failed)) { failed = true; break; }
      }
      if (tid == 0) {
        tc5::fence_after_sync();
        issue_mma_t<4>(TM_DQ, Operand{tc5::smem_addr(Do) + p * BT * 128, BT, 0}, Operand{tc5::smem_addr(Hp), DK, 0}, 64, DK, p > 0);
        issue_mma_t<4>(TM_DKS, Operand{tc5::smem_addr(Vn) + p * BT * 128, BT, 0}, Operand{tc5::smem_addr(dHp), DK, 0}, 64, DK,
                       p > 0);
        if (p == NP - 1) issue_mma_t<4>(TM_DQ, opPk, opK, 64, DK, 1);
        ph.commit();
      }
      if (p > 0) add_hd();
      if (__syncthreads_or(!ph.wait())) { failed = true; break; }
    }
    if (failed) break;

    // ---- epilogue 2: dq (this warp's half of the columns)
    // fused L2-norm backward: the finished dq stays in registers until the row dots <dq,q> are complete, so that
    // (dq - q <dq,q>) rstd is formed from the fp32 values and rounded once
    const bool l2_q = last && a.rstd_q != nullptr;
    float racc[KB][16];
    {
#pragma unroll
      for (int b = 0; b < KB; ++b) acc_ld32q(TM_DQ, q, ck + b * 32, racc[b]);
      tc5::tmem_ld_wait();
      float rq_lo = 0.f, rq_hi = 0.f;
      float rq2_lo = 0.f, rq2_hi = 0.f;   // grouped heads: the same dots for the sum over the group
#pragma unroll
      for (int b = 0; b < KB; ++b) {
        float (&r)[16] = racc[b];
        FragStore fs;
        FragLoad fq;
        fq.load(Qs, BT, q * 16, ck + b * 32, lane);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int col = ck + b * 32 + i * 8 + 2 * t;
          const float2 qa = fq.lo2(i), qb = fq.hi2(i);
          rq_lo += r[4 * i] * qa.x + r[4 * i + 1] * qa.y;
          rq_hi += r[4 * i + 2] * qb.x + r[4 * i + 3] * qb.y;
          if (GROUPED) {
            float* buf = a.dq_acc + (row0 * a.H + hq) * DK;
            const int64_t stride = (int64_t)a.H * DK;
            if (r_lo < cm.len) {
              float2* pp = reinterpret_cast<float2*>(buf + r_lo * stride + col);
              if (!first) { float2 o = *pp; r[4 * i] += o.x; r[4 * i + 1] += o.y; }
              if (!last) *pp = make_float2(r[4 * i], r[4 * i + 1]);
            }
            if (r_hi < cm.len) {
              float2* pp = reinterpret_cast<float2*>(buf + r_hi * stride + col);
              if (!first) { float2 o = *pp; r[4 * i + 2] += o.x; r[4 * i + 3] += o.y; }
              if (!last) *pp = make_float2(r[4 * i + 2], r[4 * i + 3]);
            }
          }
          if (GROUPED) {
            rq2_lo += r[4 * i] * qa.x + r[4 * i + 1] * qa.y;
            rq2_hi += r[4 * i + 2] * qb.x + r[4 * i + 3] * qb.y;
          }
          fs.set(i, r[4 * i], r[4 * i + 1], r[4 * i + 2], r[4 * i + 3]);
        }
        if (last && !l2_q) fs.store(Hp, BT, q * 16, ck + b * 32, lane);
      }
      if (GROUPED && l2_q) {
        rq2_lo += __shfl_xor_sync(0xffffffffu, rq2_lo, 1);
        rq2_lo += __shfl_xor_sync(0xffffffffu, rq2_lo, 2);
        rq2_hi += __shfl_xor_sync(0xffffffffu, rq2_hi, 1);
        rq2_hi += __shfl_xor_sync(0xffffffffu, rq2_hi, 2);
        if (t == 0) {
          rq2s[hc * BT + r_lo] = rq2_lo;
          rq2s[hc * BT + r_hi] = rq2_hi;
        }
      }
      rq_lo += __shfl_xor_sync(0xffffffffu, rq_lo, 1);
      rq_lo += __shfl_xor_sync(0xffffffffu, rq_lo, 2);
      rq_hi += __shfl_xor_sync(0xffffffffu, rq_hi, 1);
      rq_hi += __shfl_xor_sync(0xffffffffu, rq_hi, 2);
      if (t == 0) {
        rqs[hc * BT + r_lo] = rq_lo;
        rqs[hc * BT + r_hi] = rq_hi;
      }
    }
    tc5::fence_async_smem();
    tc5::fence_before_sync();
    __syncthreads();  // every warp has drained the dq columns; staging tile complete

    // ---- phase 3: dk_intra = dP~^T q (into the columns dq just left)
    if (tid == 0) {
      tc5::fence_after_sync();
      issue_mma_t<4>(TM_DKI, opPm, opQ, 64, DK, 0);
      ph.commit();
    }
    if (l2_q) {
      // q as passed is the L2-normalised tensor: dq w.r.t. the un-normalised one is (dq - q <dq,q>) rstd.  The row
      // dots are complete now (both column halves); every warp stages its block of the tile from its registers.
      const float* dots = GROUPED ? rq2s : rqs;
      const float dot_lo = dots[r_lo] + dots[BT + r_lo], dot_hi = dots[r_hi] + dots[BT + r_hi];
      const float rs_lo = r_lo < cm.len ? a.rstd_q[(row0 + r_lo) * a.H + hq] : 0.f;
      const float rs_hi = r_hi < cm.len ? a.rstd_q[(row0 + r_hi) * a.H + hq] : 0.f;
#pragma unroll
      for (int b = 0; b < KB; ++b) {
        FragLoad fq;
        fq.load(Qs, BT, q * 16, ck + b * 32, lane);
        const float (&r)[16] = racc[b];
        FragStore fs;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 qa = fq.lo2(i), qb = fq.hi2(i);
          fs.set(i, (r[4 * i] - qa.x * dot_lo) * rs_lo, (r[4 * i + 1] - qa.y * dot_lo) * rs_lo,
                 (r[4 * i + 2] - qb.x * dot_hi) * rs_hi, (r[4 * i + 3] - qb.y * dot_hi) * rs_hi);
        }
        fs.store(Hp, BT, q * 16, ck + b * 32, lane);
      }
      tc5::fence_async_smem();
      __syncthreads();
    }
    if (last) {
      if (cm.len == BT) {
        if (tid == 32) {
          tma::store_3d(&maps.dq, (int)cm.row, (hq * DK) / 64, Hp);
          tma::store_commit();
        }
      } else {
        store_tile_swz<BT, DK, NTHREADS>(reinterpret_cast<__nv_bfloat16*>(a.dq) + (row0 * a.H + hq) * DK, (int64_t)a.H * DK, Hp,
                                         cm.len, tid);
      }
    }
    if (__syncthreads_or(!ph.wait())) { failed = true; break; }

    // ---- epilogue 3: dk = dk_state + dk_intra, gate-gradient rows, tail
    {
      float rk_lo = 0.f, rk_hi = 0.f, rs = 0.f;
      float* buf = a.dk_part + (row0 * a.H + hq) * DK;
      const int64_t stride = (int64_t)a.H * DK;
      float r[KB][16], s[KB][16];
#pragma unroll
      for (int b = 0; b < KB; ++b) {
        acc_ld32q(TM_DKS, q, ck + b * 32, s[b]);
        acc_ld32q(TM_DKI, q, ck + b * 32, r[b]);
      }
      tc5::tmem_ld_wait();
      const float e_lo = fast_exp2(glast - g_lo), e_hi = fast_exp2(glast - g_hi);
#pragma unroll
      for (int b = 0; b < KB; ++b)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          s[b][4 * i] *= e_lo; s[b][4 * i + 1] *= e_lo; s[b][4 * i + 2] *= e_hi; s[b][4 * i + 3] *= e_hi;
        }
#pragma unroll
      for (int b = 0; b < KB; ++b) {
        FragStore fs;
        FragLoad fk;
        fk.load(Ks, BT, q * 16, ck + b * 32, lane);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int col = ck + b * 32 + i * 8 + 2 * t;
          const float2 ka = fk.lo2(i), kb = fk.hi2(i);
          rs += s[b][4 * i] * ka.x + s[b][4 * i + 1] * ka.y + s[b][4 * i + 2] * kb.x + s[b][4 * i + 3] * kb.y;
          const float d0 = r[b][4 * i] + s[b][4 * i], d1 = r[b][4 * i + 1] + s[b][4 * i + 1];
          const float d2 = r[b][4 * i + 2] + s[b][4 * i + 2], d3 = r[b][4 * i + 3] + s[b][4 * i + 3];
          rk_lo += d0 * ka.x + d1 * ka.y;
          rk_hi += d2 * kb.x + d3 * kb.y;
          // the value heads of a group add up in fp32 (through dk_part); the group sum leaves in bf16 through the
          // dk buffer, where the WY-backward kernel adds its terms
          float2 lo = make_float2(d0, d1), hi = make_float2(d2, d3);
          if (GROUPED) {
            if (r_lo < cm.len) {
              float2* pp = reinterpret_cast<float2*>(buf + r_lo * stride + col);
              if (!first) { const float2 o = *pp; lo.x += o.x; lo.y += o.y; }
              if (!last) *pp = lo;
            }
            if (r_hi < cm.len) {
              float2* pp = reinterpret_cast<float2*>(buf + r_hi * stride + col);
              if (!first) { const float2 o = *pp; hi.x += o.x; hi.y += o.y; }
              if (!last) *pp = hi;
            }
          }
          fs.set(i, lo.x, lo.y, hi.x, hi.y);
        }
        if (last) fs.store(dHp, BT, q * 16, ck + b * 32, lane);
      }
      rk_lo += __shfl_xor_sync(0xffffffffu, rk_lo, 1);
      rk_lo += __shfl_xor_sync(0xffffffffu, rk_lo, 2);
      rk_hi += __shfl_xor_sync(0xffffffffu, rk_hi, 1);
      rk_hi += __shfl_xor_sync(0xffffffffu, rk_hi, 2);
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        rs += __shfl_xor_sync(0xffffffffu, rs, o);
        hd += __shfl_xor_sync(0xffffffffu, hd, o);
      }
      if (lane == 0) {
        red[warp] = hd;
        red[8 + warp] = rs;
      }
      if (t == 0) {
        rks[hc * BT + r_lo] = rk_lo;
        rks[hc * BT + r_hi] = rk_hi;
      }
    }
    tc5::fence_async_smem();
    tc5::fence_before_sync();
    __syncthreads();
    if (last) {   // the chunk-local part of dk (staged over the dh panel)
      if (cm.len == BT) {
        if (tid == 32) {
          tma::store_3d(&maps.dk, (int)cm.row, (hq * DK) / 64, dHp);
          tma::store_commit();
        }
      } else {
        store_tile_swz<BT, DK, NTHREADS>(reinterpret_cast<__nv_bfloat16*>(a.dk) + (row0 * a.H + hq) * DK, (int64_t)a.H * DK, dHp,
                                         cm.len, tid);
      }
    }
    if (tid < cm.len) {
      float sh = 0.f, sr = 0.f;
#pragma unroll
      for (int w = 0; w < 8; ++w) {
        sh += red[w];
        sr += red[8 + w];
      }
      const float tail = fast_exp2(glast) * sh + sr;
      const float dGrow = (rqs[tid] + rqs[BT + tid]) - (rks[tid] + rks[BT + tid]);
      a.dG[(row0 + tid) * a.HV + hv] = dGrow + (tid == cm.len - 1 ? tail : 0.f);
    }
  }

  if (tid == 32) tma::store_wait_all<0>();   // shared memory must outlive the bulk store that reads it
  if (failed && tid == 0) atomicExch(&g_dqk_timeout, 1);
  tc5::fence_before_sync();
  __syncthreads();
  if (warp == 1) tc5::tmem_dealloc(tm, 256);
}

template <int DK, int DV, bool GROUPED>
int launch(const b200gdn_chunk_args& a, cudaStream_t st) {
  using S = DqkSmem<DK, DV>;
  if (int e = ensure_smem(bwd_dqk_kernel<DK, DV, GROUPED>, S::bytes)) return e;
  DqkMaps m;
  const uint64_t pk = (uint64_t)a.H * DK, pv = (uint64_t)a.HV * DV;
  const uint64_t hrows = (uint64_t)a.n_chunks * a.HV * DK;
  int rc = 0;
  rc |= tma::encode_bf16_panels(&m.q, a.q, a.rows, pk, pk, BT, DK / 64);
  rc |= tma::encode_bf16_panels(&m.k, a.k, a.rows, pk, pk, BT, DK / 64);
  rc |= tma::encode_bf16_panels(&m.d_o, a.d_o, a.rows, pv, pv, BT, DV / 64);
  rc |= tma::encode_bf16_panels(&m.vn, a.v_new, a.rows, pv, pv, BT, DV / 64);
  rc |= tma::encode_bf16_panels(&m.dk, a.dk, a.rows, pk, pk, BT, DK / 64);
  rc |= tma::encode_bf16_panels(&m.dq, a.dq, a.rows, pk, pk, BT, DK / 64);
  rc |= tma::encode_bf16_2d(&m.h, a.h, hrows, DV, DV, DK);
  rc |= tma::encode_bf16_2d(&m.dh, a.dh, hrows, DV, DV, DK);
  if (rc != 0) return set_error(B200GDN_ERR_CUDA, "bwd_dqk: cuTensorMapEncodeTiled failed (%d)", rc);
  dim3 grid(a.n_chunks, a.H);
  bwd_dqk_kernel<DK, DV, GROUPED><<<grid, NTHREADS, S::bytes, st>>>(a, m, resident_ctas(bwd_dqk_kernel<DK, DV, GROUPED>, NTHREADS, S::bytes));
  return check_launch("bwd_dqk");
}

}  // namespace

int launch_bwd_dqk(const b200gdn_chunk_args& a, cudaStream_t st) {
  if (a.HV > a.H && (a.dq_acc == nullptr || a.dk_part == nullptr))
    return set_error(B200GDN_ERR_BAD_ARGUMENT, "bwd_dqk: dq_acc and dk_part are required when HV > H");
  const bool grouped = a.HV > a.H;
  if (a.K == 128 && a.V == 128) return grouped ? launch<128, 128, true>(a, st) : launch<128, 128, false>(a, st);
  if (a.K == 64 && a.V == 64) return grouped ? launch<64, 64, true>(a, st) : launch<64, 64, false>(a, st);
  return set_error(B200GDN_ERR_UNSUPPORTED, "bwd_dqk: K=%d V=%d not built (64/64 and 128/128 are)", a.K, a.V);
}

// Reads and clears the flag a bounded device wait raises when it expires (synchronises with the device).
int bwd_dqk_timeout_flag() {
  int v = 0, zero = 0;
  cudaMemcpyFromSymbol(&v, g_dqk_timeout, sizeof(int));
  if (v) cudaMemcpyToSymbol(g_dqk_timeout, &zero, sizeof(int));
  return v;
}

}  // namespace gdn
