// Intra-chunk forward: gamma = cumsum(g) log2(e);  A = (I + strict_tril(beta_i <k_i,k_j> 2^(gamma_i-gamma_j)))^-1;
// W = A (K beta 2^gamma);  U = A (V beta).   One CTA of eight warps per (chunk, value head).
//
// Replaces chunk_local_cumsum (fla/ops/utils/cumsum.py:33-68), the fused K K^T + triangular solve
// (fla/ops/gated_delta_rule/chunk_fwd.py:40-328) and recompute_w_u_fwd (gated_delta_rule/wy_fast.py:43-106).
//   * K and V tiles arrive by TMA; K K^T, W and U run on tcgen05 with TMEM accumulators; A, W, U leave
//     through TMA stores (plain predicated stores for a ragged chunk);
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
__device__ int g_intra_timeout = 0;

template <int DK, int DV>
struct IntraSmem {
  static constexpr size_t o_k = 0;
  static constexpr size_t o_v = o_k + BT * DK * 2;
  static constexpr size_t o_l = o_v + BT * DV * 2;          // fp32 L ...
  static constexpr size_t o_a = o_l + sizeof(float) * BT * LDF;   // ... fp32 inverse ...
  static constexpr size_t o_t = o_a + sizeof(float) * BT * LDF;   // ... fp32 temp; the three become W | U staging
  static constexpr size_t o_aw = ((o_t + sizeof(float) * BT * LDF + 1023) / 1024) * 1024;  // bf16 A (beta 2^gamma)_col
  static constexpr size_t o_au = o_aw + BT * 128;           // bf16 A beta_col
  static constexpr size_t o_ab = o_au + BT * 128;           // bf16 A
  static constexpr size_t o_vec = o_ab + BT * 128;
  static constexpr size_t bytes = o_vec + 4 * BT * 4 + 64 + 1024;
  static constexpr size_t o_stg = ((o_l + 1023) / 1024) * 1024;   // staging for W then U (1024-aligned inside L/A/T)
  static_assert(o_stg + BT * DK * 2 + BT * DV * 2 <= o_aw, "W and U staging fit in the fp32 solve buffers");
};

struct IntraMaps {
  CUtensorMap k, v, a, w, u;
};

// T = L21 * A11 ;  A21 = -A22 * T   for an N x N off-diagonal block whose top-left corner is (r0, c0).
// `nthr` threads with local index `t` cooperate (one row x four columns each).
template <int N>
__device__ __forceinline__ void merge_step1(const float* Lf, const float* Af, float* Tf, int r0, int c0, int t, int nthr) {
  for (int o = t; o < N * N / 4; o += nthr) {
    const int i = o / (N / 4), j0 = (o % (N / 4)) * 4;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int m = 0; m < N; ++m) {
      const float l = Lf[(r0 + i) * LDF + c0 + m];
      const float4 x = *reinterpret_cast<const float4*>(&Af[(c0 + m) * LDF + c0 + j0]);
      acc[0] += l * x.x; acc[1] += l * x.y; acc[2] += l * x.z; acc[3] += l * x.w;
    }
    *reinterpret_cast<float4*>(&Tf[(r0 + i) * LDF + c0 + j0]) = make_float4(acc[0], acc[1], acc[2], acc[3]);
  }
}
template <int N>
__device__ __forceinline__ void merge_step2(const float* Tf, float* Af, int r0, int c0, int t, int nthr) {
  for (int o = t; o < N * N / 4; o += nthr) {
    const int i = o / (N / 4), j0 = (o % (N / 4)) * 4;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int m = 0; m < N; ++m) {
      const float a22 = Af[(r0 + i) * LDF + r0 + m];
      const float4 tv = *reinterpret_cast<const float4*>(&Tf[(r0 + m) * LDF + c0 + j0]);
      acc[0] += a22 * tv.x; acc[1] += a22 * tv.y; acc[2] += a22 * tv.z; acc[3] += a22 * tv.w;
    }
    *reinterpret_cast<float4*>(&Af[(r0 + i) * LDF + c0 + j0]) = make_float4(-acc[0], -acc[1], -acc[2], -acc[3]);
  }
}

template <int DK, int DV>
__global__ void __launch_bounds__(NTHREADS, 2) intra_fwd_kernel(const b200gdn_chunk_args a, const __grid_constant__ IntraMaps maps) {
  using S = IntraSmem<DK, DV>;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* Ks = smem + S::o_k;
  unsigned char* Vs = smem + S::o_v;
  float* Lf = reinterpret_cast<float*>(smem + S::o_l);
  float* Af = reinterpret_cast<float*>(smem + S::o_a);
  float* Tf = reinterpret_cast<float*>(smem + S::o_t);
  unsigned char* Aw = smem + S::o_aw;
  unsigned char* Au = smem + S::o_au;
  unsigned char* Ab = smem + S::o_ab;
  unsigned char* StgW = smem + S::o_stg;
  unsigned char* StgU = StgW + BT * DK * 2;
  float* gam = reinterpret_cast<float*>(smem + S::o_vec);
  float* bet = gam + BT;
  float* bge = bet + BT;
  float* graw = bge + BT;
  uint64_t* bar = reinterpret_cast<uint64_t*>(graw + BT);
  uint64_t* bar_ld = bar + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_ld + 1);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int q = warp & 3, hc = warp >> 2;
  const int g = lane >> 2, t = lane & 3;
  const int c = blockIdx.x, hv = blockIdx.y;
  const int G = a.HV / a.H, hq = hv / G;
  const ChunkMeta cm = load_chunk_meta(a.chunk_meta, c);
  const int64_t row0 = cm.row;
  const int r_lo = q * 16 + g, r_hi = r_lo + 8;
  const int cs = hc * 32;

  if (warp == 0) tc5::tmem_alloc(tmem_slot, 256);
  if (tid == 32) {
    tc5::mbar_init(bar, 1);
    tc5::mbar_init(bar_ld, 1);
    tc5::fence_mbar_init();
  }
  if (tid < BT) {
    const bool ok = tid < cm.len;
    graw[tid] = ok ? a.g[(row0 + tid) * a.HV + hv] : 0.f;
    bet[tid] = ok ? a.beta[(row0 + tid) * a.HV + hv] : 0.f;
  }
  // zero the fp32 inverse (upper triangles and off-diagonal blocks are read as zeros by the merges)
  for (int i = tid; i < BT * LDF; i += NTHREADS) Af[i] = 0.f;
  tc5::fence_before_sync();
  __syncthreads();
  tc5::fence_after_sync();
  const uint32_t tm = *tmem_slot;
  const uint32_t TM_KK = tm, TM_W = tm, TM_U = tm + 128;
  PhaseBarrier ph{bar, 0u, &g_intra_timeout};
  bool failed = false;

  if (tid == 0) {
    tc5::mbar_expect_tx(bar_ld, (uint32_t)(BT * DK * 2 + BT * DV * 2));
    tma::load_3d(Ks, &maps.k, cm.row, (hq * DK) / 64, bar_ld);
    tma::load_3d(Vs, &maps.v, cm.row, (hv * DV) / 64, bar_ld);
  }
  if (tid < BT) {
    // warp-shuffle inclusive scan of g over the chunk (two warps), then the cross-warp carry
    float s = graw[tid];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float y = __shfl_up_sync(0xffffffffu, s, o);
      if (lane >= o) s += y;
    }
    gam[tid] = s;
  }
  if (!tc5::mbar_wait(bar_ld, 0)) failed = true;
  if (cm.len < BT) {
    zero_tail_rows<BT, DK>(Ks, cm.len, tid, NTHREADS);
    zero_tail_rows<BT, DV>(Vs, cm.len, tid, NTHREADS);
    tc5::fence_async_smem();
  }
  if (__syncthreads_or(failed)) {
    failed = true;
  } else {
    if (tid == 0) {
      tc5::fence_after_sync();
      issue_mma_t<DK / 16>(TM_KK, Operand{tc5::smem_addr(Ks), BT, 0}, Operand{tc5::smem_addr(Ks), BT, 0}, 64, 64, 0);
      ph.commit();
    }
    if (tid < BT) {
      const float gm = (gam[tid] + (tid >= 32 ? gam[31] : 0.f)) * 1.4426950216f;
      // (the carry is read before anyone overwrites gam: see the barrier below)
      graw[tid] = gm;
    }
    __syncthreads();
    if (tid < BT) {
      const float gm = graw[tid];
      gam[tid] = gm;
      bge[tid] = bet[tid] * exp2f(gm);
      a.gamma[((int64_t)c * a.HV + hv) * BT + tid] = gm;   // padded rows carry the last valid value (their g is 0)
    }
    if (__syncthreads_or(!ph.wait())) failed = true;
  }

  if (!failed) {
    // ---- L = strict_tril(beta_i <k_i,k_j> 2^(gamma_i - gamma_j)) in fp32
    {
      float r[16];
      acc_ld32q(TM_KK, q, cs, r);
      tc5::tmem_ld_wait();
      const float g_lo = gam[r_lo], g_hi = gam[r_hi], b_lo = bet[r_lo], b_hi = bet[r_hi];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int j0 = cs + i * 8 + 2 * t;
        float v[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int ii = (e & 2) ? r_hi : r_lo, jj = j0 + (e & 1);
          v[e] = (ii > jj) ? r[4 * i + e] * ((e & 2) ? b_hi : b_lo) * exp2f(((e & 2) ? g_hi : g_lo) - gam[jj]) : 0.f;
        }
        *reinterpret_cast<float2*>(&Lf[r_lo * LDF + j0]) = make_float2(v[0], v[1]);
        *reinterpret_cast<float2*>(&Lf[r_hi * LDF + j0]) = make_float2(v[2], v[3]);
      }
    }
    tc5::fence_before_sync();
    __syncthreads();

    // ---- four 16x16 diagonal inverses: thread (block b, column cc) solves (I + L_bb) x = e_cc right-looking,
    //      so that the sixteen updates of a step are independent of each other
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
    if (tid < 128) merge_step1<16>(Lf, Af, Tf, (tid >> 6) ? 48 : 16, (tid >> 6) ? 32 : 0, tid & 63, 64);
    __syncthreads();
    if (tid < 128) merge_step2<16>(Tf, Af, (tid >> 6) ? 48 : 16, (tid >> 6) ? 32 : 0, tid & 63, 64);
    __syncthreads();
    // ---- 32 -> 64: block (32,0), all threads
    merge_step1<32>(Lf, Af, Tf, 32, 0, tid, NTHREADS);
    __syncthreads();
    merge_step2<32>(Tf, Af, 32, 0, tid, NTHREADS);
    __syncthreads();

    // ---- bf16 operand tiles: A with its columns scaled for the W and U right-hand sides, and A itself
#pragma unroll
    for (int it = 0; it < BT * BT / 2 / NTHREADS; ++it) {
      const int idx = it * NTHREADS + tid;
      const int i = idx >> 5, j = (idx & 31) * 2;
      const float2 x = *reinterpret_cast<const float2*>(&Af[i * LDF + j]);
      *swz_ptr32(Aw, i, j, BT) = pack_bf16(x.x * bge[j], x.y * bge[j + 1]);
      *swz_ptr32(Au, i, j, BT) = pack_bf16(x.x * bet[j], x.y * bet[j + 1]);
      *swz_ptr32(Ab, i, j, BT) = pack_bf16(x.x, x.y);
    }
    tc5::fence_async_smem();
    tc5::fence_before_sync();
    __syncthreads();

    // ---- W = Aw K ; U = Au V   (K and V as MN-major B operands: contraction over the token rows)
    if (tid == 0) {
      tc5::fence_after_sync();
      issue_mma_t<BT / 16>(TM_W, Operand{tc5::smem_addr(Aw), BT, 0}, Operand{tc5::smem_addr(Ks), BT, 1}, 64, DK, 0);
      issue_mma_t<BT / 16>(TM_U, Operand{tc5::smem_addr(Au), BT, 0}, Operand{tc5::smem_addr(Vs), BT, 1}, 64, DV, 0);
      ph.commit();
    }
    // A leaves while the tensor cores work
    if (cm.len == BT) {
      if (tid == 32) {
        tma::store_2d(&maps.a, hv * BT, (int)cm.row, Ab);
        tma::store_commit();
      }
    } else {
      store_tile_swz<BT, BT, NTHREADS>(reinterpret_cast<__nv_bfloat16*>(a.A) + (row0 * a.HV + hv) * BT, (int64_t)a.HV * BT, Ab,
                                       cm.len, tid);
    }
    if (__syncthreads_or(!ph.wait())) {
      failed = true;
    } else {
      constexpr int KB = DK / 64, VB = DV / 64;
      const int ck = hc * (DK / 2), cv = hc * (DV / 2);
      float rw[KB][16], ru[VB][16];
#pragma unroll
      for (int b = 0; b < KB; ++b) acc_ld32q(TM_W, q, ck + b * 32, rw[b]);
#pragma unroll
      for (int b = 0; b < VB; ++b) acc_ld32q(TM_U, q, cv + b * 32, ru[b]);
      tc5::tmem_ld_wait();
#pragma unroll
      for (int b = 0; b < KB; ++b)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int col = ck + b * 32 + i * 8 + 2 * t;
          *swz_ptr32(StgW, r_lo, col, BT) = pack_bf16(rw[b][4 * i], rw[b][4 * i + 1]);
          *swz_ptr32(StgW, r_hi, col, BT) = pack_bf16(rw[b][4 * i + 2], rw[b][4 * i + 3]);
        }
#pragma unroll
      for (int b = 0; b < VB; ++b)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int col = cv + b * 32 + i * 8 + 2 * t;
          *swz_ptr32(StgU, r_lo, col, BT) = pack_bf16(ru[b][4 * i], ru[b][4 * i + 1]);
          *swz_ptr32(StgU, r_hi, col, BT) = pack_bf16(ru[b][4 * i + 2], ru[b][4 * i + 3]);
        }
      tc5::fence_async_smem();
      tc5::fence_before_sync();
      __syncthreads();
      if (cm.len == BT) {
        if (tid == 32) {
          tma::store_3d(&maps.w, (int)cm.row, (hv * DK) / 64, StgW);
          tma::store_3d(&maps.u, (int)cm.row, (hv * DV) / 64, StgU);
          tma::store_commit();
        }
      } else {
        store_tile_swz<BT, DK, NTHREADS>(reinterpret_cast<__nv_bfloat16*>(a.w) + (row0 * a.HV + hv) * DK, (int64_t)a.HV * DK, StgW,
                                         cm.len, tid);
        store_tile_swz<BT, DV, NTHREADS>(reinterpret_cast<__nv_bfloat16*>(a.u) + (row0 * a.HV + hv) * DV, (int64_t)a.HV * DV, StgU,
                                         cm.len, tid);
      }
    }
  }
  if (tid == 32) tma::store_wait_all<0>();   // shared memory must outlive the bulk stores that read it
  if (failed && tid == 0) atomicExch(&g_intra_timeout, 1);
  tc5::fence_before_sync();
  __syncthreads();
  if (warp == 0) tc5::tmem_dealloc(tm, 256);
}

template <int DK, int DV>
int launch(const b200gdn_chunk_args& a, cudaStream_t st) {
  using S = IntraSmem<DK, DV>;
  if (int e = ensure_smem(intra_fwd_kernel<DK, DV>, S::bytes)) return e;
  IntraMaps m;
  const uint64_t pk = (uint64_t)a.H * DK, pw = (uint64_t)a.HV * DK, pv = (uint64_t)a.HV * DV, pa = (uint64_t)a.HV * BT;
  int rc = 0;
  rc |= tma::encode_bf16_panels(&m.k, a.k, a.rows, pk, pk, BT, DK / 64);
  rc |= tma::encode_bf16_panels(&m.v, a.v, a.rows, pv, pv, BT, DV / 64);
  rc |= tma::encode_bf16_2d(&m.a, a.A, a.rows, pa, pa, BT);
  rc |= tma::encode_bf16_panels(&m.w, a.w, a.rows, pw, pw, BT, DK / 64);
  rc |= tma::encode_bf16_panels(&m.u, a.u, a.rows, pv, pv, BT, DV / 64);
  if (rc != 0) return set_error(B200GDN_ERR_CUDA, "intra_fwd: cuTensorMapEncodeTiled failed (%d)", rc);
  dim3 grid(a.n_chunks, a.HV);
  intra_fwd_kernel<DK, DV><<<grid, NTHREADS, S::bytes, st>>>(a, m);
  return check_launch("intra_fwd");
}

}  // namespace

int launch_intra_fwd(const b200gdn_chunk_args& a, cudaStream_t st) {
  if (a.K == 128 && a.V == 128) return launch<128, 128>(a, st);
  if (a.K == 64 && a.V == 64) return launch<64, 64>(a, st);
  return set_error(B200GDN_ERR_UNSUPPORTED, "intra_fwd: K=%d V=%d not built (64/64 and 128/128 are)", a.K, a.V);
}

}  // namespace gdn
