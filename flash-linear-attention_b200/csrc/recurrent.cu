// Token-by-token gated delta rule (decode and short prefill), forward only:
//     S *= exp(g);  r = beta (v - S^T k);  S += k r^T;  o = S^T (scale q)
// Replaces fused_recurrent_gated_delta_rule_fwd_kernel (fla/ops/gated_delta_rule/fused_recurrent.py:30-181),
// including its in-kernel options (q/k L2 norm, -exp(A_log) softplus(g + dt_bias) gate, sigmoid beta,
// V-first state layout).  The kernel is pure state traffic at T = 1 (read K*V fp32 + write K*V fp32 per
// sequence and head), so the state is moved with 128-bit accesses, 128 contiguous bytes per 8 lanes:
// one CTA owns 32 value channels of one (sequence, head); every lane keeps 32 fp32 state elements in
// registers.  [K,V] layout: lanes run along V, the reductions over K go through registers, two shuffles
// and a 4-warp shared-memory combine.  [V,K] layout: lanes run along K and the reductions are shuffles only.
#include "gdn_common.cuh"

#include <cuda_fp16.h>

namespace gdn {
namespace {

constexpr int NTHREADS = 128;
constexpr int VS = 32;  // value channels per CTA

__device__ __forceinline__ float ld_elem(const void* p, int64_t i, int dtype) {
  if (dtype == 0) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
  if (dtype == 1) return __half2float(reinterpret_cast<const __half*>(p)[i]);
  return reinterpret_cast<const float*>(p)[i];
}
__device__ __forceinline__ void st_elem(void* p, int64_t i, int dtype, float x) {
  if (dtype == 0) reinterpret_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16(x);
  else if (dtype == 1) reinterpret_cast<__half*>(p)[i] = __float2half(x);
  else reinterpret_cast<float*>(p)[i] = x;
}
__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(expf(x)); }

template <int DK, bool VFIRST>
__global__ void __launch_bounds__(NTHREADS, (DK <= 128 ? 8 : 4)) recurrent_kernel(const b200gdn_recurrent_args a) {
  __shared__ __align__(16) float qs[DK];
  __shared__ __align__(16) float ks[DK];
  __shared__ __align__(16) float vs[VS];
  __shared__ __align__(16) float red[2][4][VS];
  __shared__ float sc[2];  // decay, beta

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int v0 = blockIdx.x * VS, hv = blockIdx.y, n = blockIdx.z;
  const int G = a.HV / a.H, hq = hv / G;
  const int DV = a.V;
  int64_t bos, len;
  if (a.cu_seqlens != nullptr) {
    bos = a.cu_seqlens[n];
    len = a.cu_seqlens[n + 1] - bos;
  } else {
    bos = (int64_t)n * a.T;
    len = a.T;
  }

  // ---- state -> registers
  // [K,V]:  st[i] holds rows  warp*(DK/4) + 4*i + lane/8  (i < DK/16), columns v0 + 4*(lane%8) .. +3
  // [V,K]:  st[p*(DK/32)+cp] holds row v0 + 8*warp + 4*p + lane/8 (p < 2), columns 32*cp + 4*(lane%8) .. +3
  constexpr int NF = DK / 16;  // float4 per lane in both layouts
  float4 st[NF];
  const int l8 = lane & 7, lg = lane >> 3;
  const float* h0 = a.h0 ? a.h0 + ((int64_t)n * a.HV + hv) * DK * DV : nullptr;
  float* ht = a.ht ? a.ht + ((int64_t)n * a.HV + hv) * DK * DV : nullptr;
  auto st_index = [&](int i) -> int64_t {
    if (!VFIRST) {
      int r = warp * (DK / 4) + 4 * i + lg;
      return (int64_t)r * DV + v0 + 4 * l8;
    } else {
      int p = i / (DK / 32), cp = i % (DK / 32);
      int r = v0 + 8 * warp + 4 * p + lg;
      return (int64_t)r * DK + 32 * cp + 4 * l8;
    }
  };
#pragma unroll
  for (int i = 0; i < NF; ++i)
    st[i] = h0 ? *reinterpret_cast<const float4*>(h0 + st_index(i)) : make_float4(0.f, 0.f, 0.f, 0.f);

  for (int64_t tok = 0; tok < len; ++tok) {
    const int64_t row = bos + tok;
    __syncthreads();  // previous token's shared inputs are no longer read
    for (int i = tid; i < DK; i += NTHREADS) {
      qs[i] = ld_elem(a.q, (row * a.H + hq) * DK + i, a.qkv_dtype);
      ks[i] = ld_elem(a.k, (row * a.H + hq) * DK + i, a.qkv_dtype);
    }
    if (tid < VS) vs[tid] = ld_elem(a.v, (row * a.HV + hv) * DV + v0 + tid, a.qkv_dtype);
    if (tid == 0) {
      float gg = a.g ? a.g[row * a.HV + hv] : 0.f;
      if (a.flags & B200GDN_REC_GATE) {
        if (a.dt_bias) gg += a.dt_bias[hv];
        gg = -expf(a.A_log[hv]) * softplus_f(gg);
      }
      float bb = a.beta[row * a.HV + hv];
      if (a.flags & B200GDN_REC_BETA_SIGMOID) {
        bb = 1.f / (1.f + expf(-bb));
        if (a.flags & B200GDN_REC_NEG_EIGVAL) bb *= 2.f;
      }
      sc[0] = expf(gg);
      sc[1] = bb;
    }
    __syncthreads();
    float qn = a.scale, kn = 1.f;
    if (a.flags & B200GDN_REC_L2NORM) {
      float sq = 0.f, sk = 0.f;
      for (int i = lane; i < DK; i += 32) {
        sq += qs[i] * qs[i];
        sk += ks[i] * ks[i];
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        sq += __shfl_xor_sync(0xffffffffu, sq, o);
        sk += __shfl_xor_sync(0xffffffffu, sk, o);
      }
      qn = a.scale * rsqrtf(sq + 1e-6f);
      kn = rsqrtf(sk + 1e-6f);
    }
    const float decay = sc[0], beta = sc[1];

    if (!VFIRST) {
      // dot over K of S and k for this lane's four columns
      float4 d = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int i = 0; i < NF; ++i) {
        st[i].x *= decay; st[i].y *= decay; st[i].z *= decay; st[i].w *= decay;
        float kk = ks[warp * (DK / 4) + 4 * i + lg] * kn;
        d.x += st[i].x * kk; d.y += st[i].y * kk; d.z += st[i].z * kk; d.w += st[i].w * kk;
      }
#pragma unroll
      for (int o = 8; o <= 16; o <<= 1) {
        d.x += __shfl_xor_sync(0xffffffffu, d.x, o);
        d.y += __shfl_xor_sync(0xffffffffu, d.y, o);
        d.z += __shfl_xor_sync(0xffffffffu, d.z, o);
        d.w += __shfl_xor_sync(0xffffffffu, d.w, o);
      }
      if (lg == 0) *reinterpret_cast<float4*>(&red[0][warp][4 * l8]) = d;
      __syncthreads();
      float4 r;
      {
        float4 s0 = *reinterpret_cast<const float4*>(&red[0][0][4 * l8]);
        float4 s1 = *reinterpret_cast<const float4*>(&red[0][1][4 * l8]);
        float4 s2 = *reinterpret_cast<const float4*>(&red[0][2][4 * l8]);
        float4 s3 = *reinterpret_cast<const float4*>(&red[0][3][4 * l8]);
        float4 vv = *reinterpret_cast<const float4*>(&vs[4 * l8]);
        r.x = beta * (vv.x - (s0.x + s1.x + s2.x + s3.x));
        r.y = beta * (vv.y - (s0.y + s1.y + s2.y + s3.y));
        r.z = beta * (vv.z - (s0.z + s1.z + s2.z + s3.z));
        r.w = beta * (vv.w - (s0.w + s1.w + s2.w + s3.w));
      }
      float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int i = 0; i < NF; ++i) {
        int rr = warp * (DK / 4) + 4 * i + lg;
        float kk = ks[rr] * kn, qq = qs[rr] * qn;
        st[i].x += kk * r.x; st[i].y += kk * r.y; st[i].z += kk * r.z; st[i].w += kk * r.w;
        o.x += st[i].x * qq; o.y += st[i].y * qq; o.z += st[i].z * qq; o.w += st[i].w * qq;
      }
#pragma unroll
      for (int of = 8; of <= 16; of <<= 1) {
        o.x += __shfl_xor_sync(0xffffffffu, o.x, of);
        o.y += __shfl_xor_sync(0xffffffffu, o.y, of);
        o.z += __shfl_xor_sync(0xffffffffu, o.z, of);
        o.w += __shfl_xor_sync(0xffffffffu, o.w, of);
      }
      if (lg == 0) *reinterpret_cast<float4*>(&red[1][warp][4 * l8]) = o;
      __syncthreads();
      if (tid < VS) {
        float s = red[1][0][tid] + red[1][1][tid] + red[1][2][tid] + red[1][3][tid];
        st_elem(a.o, (row * a.HV + hv) * DV + v0 + tid, a.qkv_dtype, s);
      }
    } else {
      constexpr int CP = DK / 32;
#pragma unroll
      for (int p = 0; p < 2; ++p) {
        const int vr = 8 * warp + 4 * p + lg;  // value channel inside the slice
        float d = 0.f;
#pragma unroll
        for (int cp = 0; cp < CP; ++cp) {
          float4& s = st[p * CP + cp];
          const float4 kk = *reinterpret_cast<const float4*>(&ks[32 * cp + 4 * l8]);
          s.x *= decay; s.y *= decay; s.z *= decay; s.w *= decay;
          d += s.x * kk.x + s.y * kk.y + s.z * kk.z + s.w * kk.w;
        }
        d *= kn;
#pragma unroll
        for (int o = 1; o <= 4; o <<= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
        const float r = beta * (vs[vr] - d) * kn;  // kn folded into the rank-one update
        float o = 0.f;
#pragma unroll
        for (int cp = 0; cp < CP; ++cp) {
          float4& s = st[p * CP + cp];
          const float4 kk = *reinterpret_cast<const float4*>(&ks[32 * cp + 4 * l8]);
          const float4 qq = *reinterpret_cast<const float4*>(&qs[32 * cp + 4 * l8]);
          s.x += r * kk.x; s.y += r * kk.y; s.z += r * kk.z; s.w += r * kk.w;
          o += s.x * qq.x + s.y * qq.y + s.z * qq.z + s.w * qq.w;
        }
        o *= qn;
#pragma unroll
        for (int of = 1; of <= 4; of <<= 1) o += __shfl_xor_sync(0xffffffffu, o, of);
        if (l8 == 0) st_elem(a.o, (row * a.HV + hv) * DV + v0 + vr, a.qkv_dtype, o);
      }
    }
  }

  if (ht != nullptr) {
#pragma unroll
    for (int i = 0; i < NF; ++i) *reinterpret_cast<float4*>(ht + st_index(i)) = st[i];
  }
}

template <int DK>
int launch(const b200gdn_recurrent_args& a, cudaStream_t st) {
  dim3 grid(a.V / VS, a.HV, a.n_seq);
  if (a.flags & B200GDN_REC_STATE_V_FIRST)
    recurrent_kernel<DK, true><<<grid, NTHREADS, 0, st>>>(a);
  else
    recurrent_kernel<DK, false><<<grid, NTHREADS, 0, st>>>(a);
  return check_launch("recurrent");
}

}  // namespace

int launch_recurrent(const b200gdn_recurrent_args& a, cudaStream_t st) {
  if (a.V % VS != 0) return set_error(B200GDN_ERR_UNSUPPORTED, "recurrent: V=%d must be a multiple of %d", a.V, VS);
  if ((a.flags & B200GDN_REC_GATE) && a.A_log == nullptr)
    return set_error(B200GDN_ERR_BAD_ARGUMENT, "recurrent: the in-kernel gate needs A_log");
  switch (a.K) {
    case 32: return launch<32>(a, st);
    case 64: return launch<64>(a, st);
    case 128: return launch<128>(a, st);
    case 256: return launch<256>(a, st);
  }
  return set_error(B200GDN_ERR_UNSUPPORTED, "recurrent: K=%d not built (32, 64, 128, 256 are)", a.K);
}

}  // namespace gdn
