// Intra-chunk forward: gamma = cumsum(g) log2(e);  A = (I + strict_tril(beta_i <k_i,k_j> 2^(gamma_i-gamma_j)))^-1;
// W = A (K beta 2^gamma);  U = A (V beta).   One CTA per (chunk, value head), four warps.
//
// Replaces chunk_local_cumsum (fla/ops/utils/cumsum.py:33-68), the fused K K^T + triangular solve
// (fla/ops/gated_delta_rule/chunk_fwd.py:40-328) and recompute_w_u_fwd (gated_delta_rule/wy_fast.py:43-106).
// The inverse is formed in fp32: the four 16x16 diagonal blocks by forward substitution (one thread per
// column), then two levels of block merges A21 = -A22 (L21 A11) (16 -> 32 -> 64).  The row scalings of
// the W/U right-hand sides are folded into the columns of A, so K and V tiles are used as loaded.
#include "gdn_common.cuh"

namespace gdn {
namespace {

constexpr int NTHREADS = 128;
constexpr int LDF = 68;  // fp32 row stride of the 64x64 solve matrices

template <int DK, int DV>
struct IntraSmem {
  static constexpr int LDK = DK + PAD, LDV = DV + PAD, LDA = BT + PAD;
  static constexpr size_t k_off = 0;
  static constexpr size_t v_off = k_off + sizeof(__nv_bfloat16) * BT * LDK;
  static constexpr size_t l_off = v_off + sizeof(__nv_bfloat16) * BT * LDV;   // fp32 L, later output staging
  static constexpr size_t a_off = l_off + sizeof(float) * BT * LDF;           // fp32 inverse
  static constexpr size_t t_off = a_off + sizeof(float) * BT * LDF;           // fp32 temp
  static constexpr size_t aw_off = t_off + sizeof(float) * BT * LDF;          // bf16 A * (beta 2^gamma)_col
  static constexpr size_t au_off = aw_off + sizeof(__nv_bfloat16) * BT * LDA; // bf16 A * beta_col
  static constexpr size_t ab_off = au_off + sizeof(__nv_bfloat16) * BT * LDA; // bf16 A (for the global store)
  static constexpr size_t vec_off = ab_off + sizeof(__nv_bfloat16) * BT * LDA;
  static constexpr size_t bytes = vec_off + sizeof(float) * 4 * BT;
  static_assert(sizeof(float) * BT * LDF * 2 >= sizeof(__nv_bfloat16) * BT * (LDK > LDV ? LDK : LDV), "staging fits");
};

// T = L21 * A11 ;  A21 = -A22 * T   for an N x N off-diagonal block whose top-left corner is (r0, c0).
// `nthr` threads with local index `t` cooperate; both steps are separated by the caller's barriers.
template <int N>
__device__ __forceinline__ void merge_step1(const float* Lf, const float* Af, float* Tf, int r0, int c0, int t, int nthr) {
  constexpr int JW = 4;
  for (int o = t; o < N * N / JW; o += nthr) {
    int i = o / (N / JW), j0 = (o % (N / JW)) * JW;
    float acc[JW] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 8
    for (int m = 0; m < N; ++m) {
      float l = Lf[(r0 + i) * LDF + c0 + m];
      float4 a = *reinterpret_cast<const float4*>(&Af[(c0 + m) * LDF + c0 + j0]);
      acc[0] += l * a.x; acc[1] += l * a.y; acc[2] += l * a.z; acc[3] += l * a.w;
    }
    *reinterpret_cast<float4*>(&Tf[(r0 + i) * LDF + c0 + j0]) = make_float4(acc[0], acc[1], acc[2], acc[3]);
  }
}
template <int N>
__device__ __forceinline__ void merge_step2(const float* Tf, float* Af, int r0, int c0, int t, int nthr) {
  constexpr int JW = 4;
  for (int o = t; o < N * N / JW; o += nthr) {
    int i = o / (N / JW), j0 = (o % (N / JW)) * JW;
    float acc[JW] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 8
    for (int m = 0; m < N; ++m) {
      float a22 = Af[(r0 + i) * LDF + r0 + m];
      float4 tv = *reinterpret_cast<const float4*>(&Tf[(r0 + m) * LDF + c0 + j0]);
      acc[0] += a22 * tv.x; acc[1] += a22 * tv.y; acc[2] += a22 * tv.z; acc[3] += a22 * tv.w;
    }
    *reinterpret_cast<float4*>(&Af[(r0 + i) * LDF + c0 + j0]) = make_float4(-acc[0], -acc[1], -acc[2], -acc[3]);
  }
}

template <int DK, int DV>
__global__ void __launch_bounds__(NTHREADS) intra_fwd_kernel(const b200gdn_chunk_args a) {
  using S = IntraSmem<DK, DV>;
  extern __shared__ __align__(16) unsigned char smem[];
  __nv_bfloat16* Ks = reinterpret_cast<__nv_bfloat16*>(smem + S::k_off);
  __nv_bfloat16* Vs = reinterpret_cast<__nv_bfloat16*>(smem + S::v_off);
  float* Lf = reinterpret_cast<float*>(smem + S::l_off);
  float* Af = reinterpret_cast<float*>(smem + S::a_off);
  float* Tf = reinterpret_cast<float*>(smem + S::t_off);
  __nv_bfloat16* Aw = reinterpret_cast<__nv_bfloat16*>(smem + S::aw_off);
  __nv_bfloat16* Au = reinterpret_cast<__nv_bfloat16*>(smem + S::au_off);
  __nv_bfloat16* Ab = reinterpret_cast<__nv_bfloat16*>(smem + S::ab_off);
  float* gam = reinterpret_cast<float*>(smem + S::vec_off);  // gamma
  float* bet = gam + BT;                                      // beta
  float* bge = bet + BT;                                      // beta * 2^gamma
  float* graw = bge + BT;
  __nv_bfloat16* stage = reinterpret_cast<__nv_bfloat16*>(smem + S::l_off);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int c = blockIdx.x, hv = blockIdx.y;
  const int G = a.HV / a.H, hq = hv / G;
  const ChunkMeta cm = load_chunk_meta(a.chunk_meta, c);
  const int64_t row0 = cm.row;

  const __nv_bfloat16* kg = reinterpret_cast<const __nv_bfloat16*>(a.k) + (row0 * a.H + hq) * DK;
  const __nv_bfloat16* vg = reinterpret_cast<const __nv_bfloat16*>(a.v) + (row0 * a.HV + hv) * DV;
  load_tile_async<DK, NTHREADS>(Ks, kg, (int64_t)a.H * DK, cm.len, tid);
  load_tile_async<DV, NTHREADS>(Vs, vg, (int64_t)a.HV * DV, cm.len, tid);
  cp_async_commit();
  if (tid < BT) {
    bool ok = tid < cm.len;
    graw[tid] = ok ? a.g[(row0 + tid) * a.HV + hv] : 0.f;
    bet[tid] = ok ? a.beta[(row0 + tid) * a.HV + hv] : 0.f;
  }
  // zero the fp32 inverse (upper triangles and off-diagonal blocks are read as zeros by the merges)
  for (int i = tid; i < BT * LDF; i += NTHREADS) Af[i] = 0.f;
  __syncthreads();
  if (tid < BT) {
    float s = 0.f;
    for (int j = 0; j <= tid; ++j) s += graw[j];
    float gm = s * 1.4426950216f;
    gam[tid] = gm;
    bge[tid] = bet[tid] * exp2f(gm);
    a.gamma[((int64_t)c * a.HV + hv) * BT + tid] = gm;   // padded rows carry the last valid value (their g is 0)
  }
  cp_async_wait<0>();
  __syncthreads();

  // ---- L = strict_tril(beta_i <k_i,k_j> 2^(gamma_i - gamma_j)) in fp32
  {
    float acc[8][4];
    zero_acc<8>(acc);
    warp_mma<8, DK / 16, AMajor::Row, BMajor::NK>(acc, Ks + warp * 16 * S::LDK, S::LDK, Ks, S::LDK, lane);
    const int g = lane >> 2, t = lane & 3;
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        int i = warp * 16 + g + ((e >> 1) << 3);
        int j = nt * 8 + 2 * t + (e & 1);
        float val = 0.f;
        if (i > j) val = bet[i] * acc[nt][e] * exp2f(gam[i] - gam[j]);  // mask first: the exponent overflows above the diagonal
        Lf[i * LDF + j] = val;
      }
    }
  }
  __syncthreads();

  // ---- diagonal 16x16 blocks: column c of (I + L_bb)^-1 by forward substitution
  if (tid < BT) {
    const int b = tid >> 4, col = tid & 15;
    float x[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      float s = (i == col) ? 1.f : 0.f;
#pragma unroll
      for (int j = 0; j < i; ++j) s -= Lf[(b * 16 + i) * LDF + b * 16 + j] * x[j];
      x[i] = s;
    }
#pragma unroll
    for (int i = 0; i < 16; ++i) Af[(b * 16 + i) * LDF + b * 16 + col] = x[i];
  }
  __syncthreads();
  // ---- 16 -> 32: two independent merges, 64 threads each
  {
    const int half = tid >> 6, t = tid & 63;
    merge_step1<16>(Lf, Af, Tf, half * 32 + 16, half * 32, t, 64);
    __syncthreads();
    merge_step2<16>(Tf, Af, half * 32 + 16, half * 32, t, 64);
    __syncthreads();
  }
  // ---- 32 -> 64
  merge_step1<32>(Lf, Af, Tf, 32, 0, tid, NTHREADS);
  __syncthreads();
  merge_step2<32>(Tf, Af, 32, 0, tid, NTHREADS);
  __syncthreads();

  // ---- bf16 copies of A: plain (saved for the backward pass) and column-scaled (operands of W and U)
  for (int idx = tid; idx < BT * BT / 2; idx += NTHREADS) {
    int i = idx / (BT / 2), j = (idx % (BT / 2)) * 2;
    float a0 = Af[i * LDF + j], a1 = Af[i * LDF + j + 1];
    *reinterpret_cast<uint32_t*>(&Ab[i * S::LDA + j]) = pack_bf16(a0, a1);
    *reinterpret_cast<uint32_t*>(&Aw[i * S::LDA + j]) = pack_bf16(a0 * bge[j], a1 * bge[j + 1]);
    *reinterpret_cast<uint32_t*>(&Au[i * S::LDA + j]) = pack_bf16(a0 * bet[j], a1 * bet[j + 1]);
  }
  __syncthreads();
  store_tile<BT, BT, NTHREADS>(reinterpret_cast<__nv_bfloat16*>(a.A) + (row0 * a.HV + hv) * BT, (int64_t)a.HV * BT, Ab,
                               cm.len, tid);

  // ---- W = Aw K
  {
    float acc[DK / 8][4];
    zero_acc<DK / 8>(acc);
    warp_mma<DK / 8, BT / 16, AMajor::Row, BMajor::KN>(acc, Aw + warp * 16 * S::LDA, S::LDA, Ks, S::LDK, lane);
    acc_to_smem<DK / 8>(stage + warp * 16 * S::LDK, S::LDK, acc, lane);  // Lf/Af region: free since the barrier above
  }
  __syncthreads();
  store_tile<BT, DK, NTHREADS>(reinterpret_cast<__nv_bfloat16*>(a.w) + (row0 * a.HV + hv) * DK, (int64_t)a.HV * DK, stage,
                               cm.len, tid);
  __syncthreads();
  // ---- U = Au V
  {
    float acc[DV / 8][4];
    zero_acc<DV / 8>(acc);
    warp_mma<DV / 8, BT / 16, AMajor::Row, BMajor::KN>(acc, Au + warp * 16 * S::LDA, S::LDA, Vs, S::LDV, lane);
    acc_to_smem<DV / 8>(stage + warp * 16 * S::LDV, S::LDV, acc, lane);
  }
  __syncthreads();
  store_tile<BT, DV, NTHREADS>(reinterpret_cast<__nv_bfloat16*>(a.u) + (row0 * a.HV + hv) * DV, (int64_t)a.HV * DV, stage,
                               cm.len, tid);
}

template <int DK, int DV>
int launch(const b200gdn_chunk_args& a, cudaStream_t st) {
  using S = IntraSmem<DK, DV>;
  if (int e = ensure_smem(intra_fwd_kernel<DK, DV>, S::bytes)) return e;
  dim3 grid(a.n_chunks, a.HV);
  intra_fwd_kernel<DK, DV><<<grid, NTHREADS, S::bytes, st>>>(a);
  return check_launch("intra_fwd");
}

}  // namespace

int launch_intra_fwd(const b200gdn_chunk_args& a, cudaStream_t st) {
  if (a.K == 128 && a.V == 128) return launch<128, 128>(a, st);
  if (a.K == 64 && a.V == 64) return launch<64, 64>(a, st);
  return set_error(B200GDN_ERR_UNSUPPORTED, "intra_fwd: K=%d V=%d not built (64/64 and 128/128 are)", a.K, a.V);
}

}  // namespace gdn
