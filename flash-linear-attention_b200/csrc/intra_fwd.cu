// Intra-chunk forward: gamma = cumsum(g) log2(e);  A = (I + strict_tril(beta_i <k_i,k_j> 2^(gamma_i-gamma_j)))^-1;
// W = A (K beta 2^gamma);  U = A (V beta);  and (when q and a qk buffer are given)
// qk = tril(<q_i,k_j> 2^(gamma_i-gamma_j)), the chunk-local attention tile of chunk_fwd_kernel_o /
// chunk_bwd_kernel_dv_local (fla/ops/common/chunk_o.py:115-127, 505-520), which shares K, gamma and the gate factors
// with L.   One CTA of eight warps per (chunk, value head).
//
// Replaces chunk_local_cumsum (fla/ops/utils/cumsum.py:33-68), the fused K K^T + triangular solve
// (fla/ops/gated_delta_rule/chunk_fwd.py:40-328) and recompute_w_u_fwd (gated_delta_rule/wy_fast.py:43-106).
//   * K and V tiles arrive by TMA; K K^T, W and U run on tcgen05 with TMEM accumulators (128 columns, used
//     one product after the other); A, W, U leave through TMA stores (plain predicated stores for a ragged
//     chunk); shared-memory regions are reused along the way so that three CTAs share an SM and hide each
//     other's latencies;
//   * the inverse is formed in exact fp32 on the CUDA cores: the four 16x16 diagonal blocks by
//     right-looking forward substitution (one thread per column), then two levels of block merges
//     A21 = -A22 (L21 A11) (16 -> 32 -> 64); the reference uses tf32 tensor-core merges;
//   * the row scalings of the W/U right-hand sides are folded into the columns of A, so the K and V
//     tiles are used exactly as loaded.
#include "tc5_tile.cuh"
#include "tma.cuh"

namespace gdn {
namespace {

constexpr int NTHREADS = 256;
constexpr int LDF = 68;  // fp32 row stride of the 64x64 solve matrices
constexpr int LDT = 36;  // fp32 row stride of the (at most 32x32) merge temporary
__device__ int g_intra_timeout = 0;

template <int DK, int DV>
struct IntraSmem {
  // Regions are reused as the kernel advances (each hand-over is separated by a CTA barrier):
  //   K tile                      -> W staging
  //   fp32 L                      -> V tile (loaded once L is dead) -> U staging
  //   fp32 inverse                -> bf16 A (beta 2^gamma)_col | A beta_col
  //   fp32 merge temporary (32x32)
  // 56 896 bytes at K = V = 128: with the 1 KiB the system keeps per CTA, four CTAs fill the 228 KiB of an SM exactly,
  // which is why the dynamic window is used from its (1024-byte aligned, checked) start without an alignment slack.
  static constexpr size_t fmat = ((sizeof(float) * BT * LDF + 1023) / 1024) * 1024;
  static constexpr size_t o_k = 0;
  static constexpr size_t o_l = o_k + BT * DK * 2;
  static constexpr size_t o_a = o_l + (fmat > BT * DV * 2 ? fmat : BT * DV * 2);
  static constexpr size_t o_t = o_a + fmat;
  static constexpr size_t o_vec = o_t + sizeof(float) * 32 * LDT;
  static constexpr size_t bytes = o_vec + 4 * BT * 4 + 64;
  static_assert(fmat >= 2 * BT * 128, "two bf16 64x64 tiles fit in the fp32 inverse");
  static_assert((sizeof(float) * 32 * LDT) % 16 == 0, "vectors stay 16-byte aligned");
};

struct IntraMaps {
  CUtensorMap k, v, w, u, q;
};

// T = L21 * A11 ;  A21 = -A22 * T   for an N x N off-diagonal block whose top-left corner is (r0, c0).
// T is kept in a compact temporary (row stride LDT).  `nthr` threads with local index `t` cooperate
// (one row x four columns each).
template <int N>
__device__ __forceinline__ void merge_step1(const float* Lf, const float* Af, float* T, int r0, int c0, int t, int nthr) {
  for (int o = t; o < N * N / 4; o += nthr) {
    const int i = o / (N / 4), j0 = (o % (N / 4)) * 4;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int m = 0; m < N; ++m) {
      const float l = Lf[(r0 + i) * LDF + c0 + m];
      const float4 x = *reinterpret_cast<const float4*>(&Af[(c0 + m) * LDF + c0 + j0]);
      acc[0] += l * x.x; acc[1] += l * x.y; acc[2] += l * x.z; acc[3] += l * x.w;
    }
    *reinterpret_cast<float4*>(&T[i * LDT + j0]) = make_float4(acc[0], acc[1], acc[2], acc[3]);
  }
}
// A22 is lower triangular, so row i only needs m <= i; `m_end` is that bound rounded up to something uniform over
// the calling warp (the rows of a warp are consecutive), which keeps the loop free of divergence.
template <int N>
__device__ __forceinline__ void merge_step2(const float* T, float* Af, int r0, int c0, int t, int nthr, int m_end) {
  for (int o = t; o < N * N / 4; o += nthr) {
    const int i = o / (N / 4), j0 = (o % (N / 4)) * 4;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 4
    for (int m = 0; m < m_end; ++m) {
      const float a22 = Af[(r0 + i) * LDF + r0 + m];
      const float4 tv = *reinterpret_cast<const float4*>(&T[m * LDT + j0]);
      acc[0] += a22 * tv.x; acc[1] += a22 * tv.y; acc[2] += a22 * tv.z; acc[3] += a22 * tv.w;
    }
    *reinterpret_cast<float4*>(&Af[(r0 + i) * LDF + c0 + j0]) = make_float4(-acc[0], -acc[1], -acc[2], -acc[3]);
  }
}

template <int DK, int DV>
__global__ void __launch_bounds__(NTHREADS, 4) intra_fwd_kernel(const b200gdn_chunk_args a, const __grid_constant__ IntraMaps maps,
                                                                const int pf_dist) {
  using S = IntraSmem<DK, DV>;
  constexpr int KB = DK / 64, VB = DV / 64;
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* smem = smem_raw;
  if ((tc5::smem_addr(smem) & 1023u) != 0) {   // the swizzled tiles need it; never seen, but never silently wrong either
    if (threadIdx.x == 0) atomicExch(&g_intra_timeout, 2);
    return;
  }
  unsigned char* Ks = smem + S::o_k;      // later the W staging tile
  unsigned char* Vs = smem + S::o_l;      // after L; later the U staging tile
  float* Lf = reinterpret_cast<float*>(smem + S::o_l);
  float* Af = reinterpret_cast<float*>(smem + S::o_a);
  float* Tf = reinterpret_cast<float*>(smem + S::o_t);
  unsigned char* Aw = smem + S::o_a;      // after the fp32 inverse has been read into registers
  unsigned char* Au = Aw + BT * 128;
  float* gam = reinterpret_cast<float*>(smem + S::o_vec);
  float* bet = gam + BT;
  float* bge = bet + BT;
  float* graw = bge + BT;
  uint64_t* bar = reinterpret_cast<uint64_t*>(graw + BT);
  uint64_t* bar_k = bar + 1;
  uint64_t* bar_v = bar + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar + 3);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int q = warp & 3, hc = warp >> 2;
  const int g = lane >> 2, t = lane & 3;
  const int c = blockIdx.x, hv = blockIdx.y;
  const int G = a.HV / a.H, hq = hv / G;
  const ChunkMeta cm = load_chunk_meta(a.chunk_meta, c);
  const int64_t row0 = cm.row;
  const int r_lo = q * 16 + g, r_hi = r_lo + 8;
  const int cs = hc * 32;
  // with q and a qk buffer the kernel also emits the gated causal q k^T tile that the scans use for the chunk-local
  // parts of o and dv (so that they neither form nor mask it on their serial chain)
  const bool with_qk = a.qk != nullptr && a.q != nullptr;
  unsigned char* Qs = smem + S::o_l;

  if (tid == 0) {
    tc5::mbar_init(bar, 1);
    tc5::mbar_init(bar_k, 1);
    tc5::mbar_init(bar_v, 1);
    tc5::fence_mbar_init();
    tc5::mbar_expect_tx(bar_k, (uint32_t)((with_qk ? 2 : 1) * BT * DK * 2));
    tma::load_3d(Ks, &maps.k, cm.row, (hq * DK) / 64, bar_k);
    if (with_qk) tma::load_3d(Qs, &maps.q, cm.row, (hq * DK) / 64, bar_k);   // lives where L will be written
    tma::prefetch_3d(&maps.v, cm.row, (hv * DV) / 64);   // V is loaded late (it reuses L's place): have it in L2 by then
  }
  if (warp == 1) tc5::tmem_alloc(tmem_slot, 128);
  if (tid < BT) {   // asynchronous copies: nobody stalls on the DRAM latency of the gates before the first barrier
    if (tid < cm.len) {
      cp_async4(graw + tid, a.g + (row0 + tid) * a.HV + hv);
      cp_async4(bet + tid, a.beta + (row0 + tid) * a.HV + hv);
    } else {
      graw[tid] = 0.f;
      bet[tid] = 0.f;
    }
    cp_async_commit();
  }
  // zero the fp32 inverse (the merges and the final conversion read the untouched blocks as zeros)
  for (int i = tid; i < BT * LDF / 4; i += NTHREADS) reinterpret_cast<float4*>(Af)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
  tc5::fence_before_sync();
  __syncthreads();
  tc5::fence_after_sync();
  const uint32_t tm = *tmem_slot;
  PhaseBarrier ph{bar, 0u, &g_intra_timeout};
  bool failed = false;

  if (tid < BT) {
    // inclusive scan of g over the chunk: shuffle scan inside each of the two warps, carry added below
    cp_async_wait<0>();   // this thread's own g and beta
    if (a.options != 0 && tid < cm.len) {   // the layer's gate / beta activations, fused (rows past the end stay 0)
      if (a.options & B200GDN_PREP_GATE) {
        const float x = graw[tid] + (a.dt_bias ? a.dt_bias[hv] : 0.f);
        graw[tid] = -expf(a.A_log[hv]) * (x > 20.f ? x : log1pf(expf(x)));
      }
      if (a.options & B200GDN_PREP_BETA_SIGMOID)
        bet[tid] = ((a.options & B200GDN_PREP_NEG_EIGVAL) ? 2.f : 1.f) / (1.f + expf(-bet[tid]));
    }
    float s = graw[tid];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float y = __shfl_up_sync(0xffffffffu, s, o);
      if (lane >= o) s += y;
    }
    gam[tid] = s;
  }
  if (tid == 128) {   // while everybody waits for the K tile
    int c2, h2;
    if (successor_cta(pf_dist, c2, h2)) {   // L2 look-ahead for the CTA that will follow this one
      const int row2 = load_chunk_meta(a.chunk_meta, c2).row;
      tma::prefetch_3d(&maps.k, row2, ((h2 / G) * DK) / 64);
      // g and beta of a chunk are [64][HV] fp32 blocks: the HV CTAs of a chunk pull two lines each
      const int lines = BT * a.HV * 4 / 128;
      for (int l = h2 * 2; l < h2 * 2 + 2 && l < lines; ++l) {
        tma::prefetch_line(a.g + (int64_t)row2 * a.HV + l * 32);
        tma::prefetch_line(a.beta + (int64_t)row2 * a.HV + l * 32);
      }
    }
  }
  if (!tc5::mbar_wait(bar_k, 0)) failed = true;
  if (cm.len < BT) {
    zero_tail_rows<BT, DK>(Ks, cm.len, tid, NTHREADS);
    tc5::fence_async_smem();
  }
  if (__syncthreads_or(failed)) {
    failed = true;
  } else {
    if (tid == 0) {
      tc5::fence_after_sync();
      issue_mma_t<DK / 16>(tm, Operand{tc5::smem_addr(Ks), BT, 0}, Operand{tc5::smem_addr(Ks), BT, 0}, 64, 64, 0);
      if (with_qk) issue_mma_t<DK / 16>(tm + 64, Operand{tc5::smem_addr(Qs), BT, 0}, Operand{tc5::smem_addr(Ks), BT, 0}, 64, 64, 0);
      ph.commit();
    }
    if (tid < BT) graw[tid] = (gam[tid] + (tid >= 32 ? gam[31] : 0.f)) * 1.4426950216f;
    __syncthreads();
    if (tid < BT) {
      // entries past a ragged chunk's end repeat the last valid value exactly (the scan sums zeros there, but in an
      // order that depends on the lane, so its result may differ in the last bit)
      const float gm = graw[tid < cm.len ? tid : cm.len - 1];
      gam[tid] = gm;
      bge[tid] = bet[tid] * fast_exp2(gm);
      a.gamma[((int64_t)c * a.HV + hv) * BT + tid] = gm;   // padded rows carry the last valid value (their g is 0)
    }
    if (!ph.sync_wait()) failed = true;
  }

  if (!failed) {
    // ---- L = strict_tril(beta_i <k_i,k_j> 2^(gamma_i - gamma_j)) in fp32 (over the Q tile, which is dead by now), and
    //      qk = tril(<q_i,k_j> 2^(gamma_i - gamma_j)) with the same gate factors, as bf16 straight to global memory
    //      (rows past a ragged chunk's end are another sequence's rows and are not written)
    {
      __nv_bfloat16* Pg = reinterpret_cast<__nv_bfloat16*>(a.qk) + (row0 * a.HV + hv) * BT + cs + 2 * t;
      const int64_t pstride = (int64_t)a.HV * BT;
      if (q * 16 + 15 >= cs) {   // a block entirely above the diagonal is never read by the solve and is zero in qk
        float r[16], pq[16];
        acc_ld32q(tm, q, cs, r);
        if (with_qk) acc_ld32q(tm + 64, q, cs, pq);
        tc5::tmem_ld_wait();
        const float g_lo = gam[r_lo], g_hi = gam[r_hi], b_lo = bet[r_lo], b_hi = bet[r_hi];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int j0 = cs + i * 8 + 2 * t;
          float v[4], w4[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int ii = (e & 2) ? r_hi : r_lo, jj = j0 + (e & 1);
            const float f = fast_exp2(((e & 2) ? g_hi : g_lo) - gam[jj]);
            v[e] = (ii > jj) ? r[4 * i + e] * ((e & 2) ? b_hi : b_lo) * f : 0.f;
            w4[e] = (with_qk && ii >= jj) ? pq[4 * i + e] * f : 0.f;
          }
          *reinterpret_cast<float2*>(&Lf[r_lo * LDF + j0]) = make_float2(v[0], v[1]);
          *reinterpret_cast<float2*>(&Lf[r_hi * LDF + j0]) = make_float2(v[2], v[3]);
          if (with_qk) {
            if (r_lo < cm.len) *reinterpret_cast<uint32_t*>(Pg + r_lo * pstride + i * 8) = pack_bf16(w4[0], w4[1]);
            if (r_hi < cm.len) *reinterpret_cast<uint32_t*>(Pg + r_hi * pstride + i * 8) = pack_bf16(w4[2], w4[3]);
          }
        }
      } else if (with_qk) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          if (r_lo < cm.len) *reinterpret_cast<uint32_t*>(Pg + r_lo * pstride + i * 8) = 0u;
          if (r_hi < cm.len) *reinterpret_cast<uint32_t*>(Pg + r_hi * pstride + i * 8) = 0u;
        }
      }
    }
    tc5::fence_before_sync();
    __syncthreads();

    // ---- four 16x16 diagonal inverses: thread (block b, column cc) solves (I + L_bb) x = e_cc right-looking,
    //      so that the updates of one step are independent of each other
    if (tid < BT) {
      const int b0 = (tid >> 4) * 16, cc = tid & 15;
      float s[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) s[i] = (i == cc) ? 1.f : 0.f;
#pragma unroll
      for (int j = 0; j < 15; ++j) {
        const float xj = s[j];
#pragma unroll
        for (int i = j + 1; i < 16; ++i) s[i] -= Lf[(b0 + i) * LDF + b0 + j] * xj;
      }
#pragma unroll
      for (int i = 0; i < 16; ++i) Af[(b0 + i) * LDF + b0 + cc] = s[i];
    }
    __syncthreads();
    // ---- 16 -> 32: blocks (16,0) and (48,32), 64 threads each
    if (tid < 128) merge_step1<16>(Lf, Af, Tf + (tid >> 6) * 16, (tid >> 6) ? 48 : 16, (tid >> 6) ? 32 : 0, tid & 63, 64);
    __syncthreads();
    if (tid < 128) merge_step2<16>(Tf + (tid >> 6) * 16, Af, (tid >> 6) ? 48 : 16, (tid >> 6) ? 32 : 0, tid & 63, 64, 8 * (warp & 1) + 8);
    __syncthreads();
    // ---- 32 -> 64: block (32,0), all threads
    merge_step1<32>(Lf, Af, Tf, 32, 0, tid, NTHREADS);
    __syncthreads();
    // L is dead: its place takes the V tile while the last merge step and the conversion run
    if (tid == 0) {
      tc5::fence_async_smem();
      tc5::mbar_expect_tx(bar_v, (uint32_t)(BT * DV * 2));
      tma::load_3d(Vs, &maps.v, cm.row, (hv * DV) / 64, bar_v);
    }
    merge_step2<32>(Tf, Af, 32, 0, tid, NTHREADS, 4 * warp + 4);
    __syncthreads();

    // ---- bf16 operand tiles (over the fp32 inverse and the merge temporary, hence through registers):
    //      A with its columns scaled for the W and U right-hand sides, and A itself
    {   // every warp converts its own 16 x 32 block (rows 16 q .., columns cs ..) in the accumulator-fragment layout
      float2 x_lo[4], x_hi[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int col = cs + i * 8 + 2 * t;
        x_lo[i] = *reinterpret_cast<const float2*>(&Af[r_lo * LDF + col]);
        x_hi[i] = *reinterpret_cast<const float2*>(&Af[r_hi * LDF + col]);
      }
      __syncthreads();
      FragStore fw, fu, fa;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int col = cs + i * 8 + 2 * t;
        const float2 sw = *reinterpret_cast<const float2*>(&bge[col]), su = *reinterpret_cast<const float2*>(&bet[col]);
        fw.set(i, x_lo[i].x * sw.x, x_lo[i].y * sw.y, x_hi[i].x * sw.x, x_hi[i].y * sw.y);
        fu.set(i, x_lo[i].x * su.x, x_lo[i].y * su.y, x_hi[i].x * su.x, x_hi[i].y * su.y);
        fa.set(i, x_lo[i].x, x_lo[i].y, x_hi[i].x, x_hi[i].y);
      }
      fw.store(Aw, BT, q * 16, cs, lane);
      fu.store(Au, BT, q * 16, cs, lane);
      // A itself goes straight to global memory (16 contiguous bytes per lane quad and row)
      __nv_bfloat16* Ag = reinterpret_cast<__nv_bfloat16*>(a.A) + (row0 * a.HV + hv) * BT + cs + 2 * t;
      const int64_t astride = (int64_t)a.HV * BT;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        if (r_lo < cm.len) *reinterpret_cast<uint32_t*>(Ag + r_lo * astride + i * 8) = fa.lo[i];
        if (r_hi < cm.len) *reinterpret_cast<uint32_t*>(Ag + r_hi * astride + i * 8) = fa.hi[i];
      }
    }
    tc5::fence_async_smem();
    tc5::fence_before_sync();
    __syncthreads();

    // ---- W = Aw K   (K as an MN-major B operand: contraction over the token rows)
    if (tid == 0) {
      tc5::fence_after_sync();
      issue_mma_t<BT / 16>(tm, Operand{tc5::smem_addr(Aw), BT, 0}, Operand{tc5::smem_addr(Ks), BT, 1}, 64, DK, 0);
      ph.commit();
    }
    if (!tc5::mbar_wait(bar_v, 0)) failed = true;
    if (cm.len < BT) {
      zero_tail_rows<BT, DV>(Vs, cm.len, tid, NTHREADS);
      tc5::fence_async_smem();
    }
    if (!ph.sync_wait(failed)) {
      failed = true;
    } else {
      const int ck = hc * (DK / 2), cv = hc * (DV / 2);
      float rw[KB][16];
#pragma unroll
      for (int b = 0; b < KB; ++b) acc_ld32q(tm, q, ck + b * 32, rw[b]);
      tc5::tmem_ld_wait();
      tc5::fence_before_sync();
      __syncthreads();   // W has left tensor memory, K is no longer an operand
      // ---- U = Au V into the same columns, while W is converted and staged over the K tile
      if (tid == 0) {
        tc5::fence_after_sync();
        issue_mma_t<BT / 16>(tm, Operand{tc5::smem_addr(Au), BT, 0}, Operand{tc5::smem_addr(Vs), BT, 1}, 64, DV, 0);
        ph.commit();
      }
#pragma unroll
      for (int b = 0; b < KB; ++b) {
        FragStore fs;
#pragma unroll
        for (int i = 0; i < 4; ++i) fs.set(i, rw[b][4 * i], rw[b][4 * i + 1], rw[b][4 * i + 2], rw[b][4 * i + 3]);
        fs.store(Ks, BT, q * 16, ck + b * 32, lane);
      }
      tc5::fence_async_smem();
      if (!ph.sync_wait()) {
        failed = true;
      } else {
        if (cm.len == BT) {
          if (tid == 32) {
            tma::store_3d(&maps.w, (int)cm.row, (hv * DK) / 64, Ks);
            tma::store_commit();
          }
        } else {
          store_tile_swz<BT, DK, NTHREADS>(reinterpret_cast<__nv_bfloat16*>(a.w) + (row0 * a.HV + hv) * DK, (int64_t)a.HV * DK,
                                           Ks, cm.len, tid);
        }
        float ru[VB][16];
#pragma unroll
        for (int b = 0; b < VB; ++b) acc_ld32q(tm, q, cv + b * 32, ru[b]);
        tc5::tmem_ld_wait();
#pragma unroll
        for (int b = 0; b < VB; ++b) {
          FragStore fs;
#pragma unroll
          for (int i = 0; i < 4; ++i) fs.set(i, ru[b][4 * i], ru[b][4 * i + 1], ru[b][4 * i + 2], ru[b][4 * i + 3]);
          fs.store(Vs, BT, q * 16, cv + b * 32, lane);
        }
        tc5::fence_async_smem();
        tc5::fence_before_sync();
        __syncthreads();
        if (cm.len == BT) {
          if (tid == 32) {
            tma::store_3d(&maps.u, (int)cm.row, (hv * DV) / 64, Vs);
            tma::store_commit();
          }
        } else {
          store_tile_swz<BT, DV, NTHREADS>(reinterpret_cast<__nv_bfloat16*>(a.u) + (row0 * a.HV + hv) * DV, (int64_t)a.HV * DV,
                                           Vs, cm.len, tid);
        }
      }
    }
  }
  if (tid == 32) tma::store_wait_all<0>();   // shared memory must outlive the bulk stores that read it
  if (failed && tid == 0) atomicExch(&g_intra_timeout, 1);
  tc5::fence_before_sync();
  __syncthreads();
  if (warp == 1) tc5::tmem_dealloc(tm, 128);
}

template <int DK, int DV>
int launch(const b200gdn_chunk_args& a, cudaStream_t st) {
  using S = IntraSmem<DK, DV>;
  if (int e = ensure_smem(intra_fwd_kernel<DK, DV>, S::bytes)) return e;
  IntraMaps m;
  const uint64_t pk = (uint64_t)a.H * DK, pw = (uint64_t)a.HV * DK, pv = (uint64_t)a.HV * DV;
  int rc = 0;
  rc |= tma::encode_bf16_panels(&m.k, a.k, a.rows, pk, pk, BT, DK / 64);
  rc |= tma::encode_bf16_panels(&m.v, a.v, a.rows, pv, pv, BT, DV / 64);
  rc |= tma::encode_bf16_panels(&m.w, a.w, a.rows, pw, pw, BT, DK / 64);
  rc |= tma::encode_bf16_panels(&m.u, a.u, a.rows, pv, pv, BT, DV / 64);
  if (a.q) rc |= tma::encode_bf16_panels(&m.q, a.q, a.rows, pk, pk, BT, DK / 64); else m.q = m.k;
  if (rc != 0) return set_error(B200GDN_ERR_CUDA, "intra_fwd: cuTensorMapEncodeTiled failed (%d)", rc);
  dim3 grid(a.n_chunks, a.HV);
  intra_fwd_kernel<DK, DV><<<grid, NTHREADS, S::bytes, st>>>(a, m, resident_ctas(intra_fwd_kernel<DK, DV>, NTHREADS, S::bytes));
  return check_launch("intra_fwd");
}

}  // namespace

int launch_intra_fwd(const b200gdn_chunk_args& a, cudaStream_t st) {
  if ((a.options & B200GDN_PREP_GATE) && a.A_log == nullptr)
    return set_error(B200GDN_ERR_BAD_ARGUMENT, "intra_fwd: the fused gate needs A_log");
  if (a.K == 128 && a.V == 128) return launch<128, 128>(a, st);
  if (a.K == 64 && a.V == 64) return launch<64, 64>(a, st);
  return set_error(B200GDN_ERR_UNSUPPORTED, "intra_fwd: K=%d V=%d not built (64/64 and 128/128 are)", a.K, a.V);
}

// Reads and clears the flag a bounded device wait raises when it expires (synchronises with the device).
int intra_fwd_timeout_flag() {
  int v = 0, zero = 0;
  cudaMemcpyFromSymbol(&v, g_intra_timeout, sizeof(int));
  if (v) cudaMemcpyToSymbol(g_intra_timeout, &zero, sizeof(int));
  return v;
}

}  // namespace gdn
