// The layer's three element-wise options as one pass before the chunk kernels and one pass after their backward:
// L2 normalisation of q and k over the key dimension (fla/modules/l2norm.py:84-144), the gate activation
// -exp(A_log) softplus(g + dt_bias) with its parameter gradients (fla/ops/gated_delta_rule/gate.py:63-158) and
// beta = s sigmoid(.) (fla/ops/common/gate.py:18-50).  Pure HBM streaming: every kernel moves 16 bytes per
// thread and access; one warp owns one (token, head) vector of K elements.
#include <cuda_fp16.h>

#include "gdn_common.cuh"
#include "rowio.cuh"

namespace gdn {
namespace {

constexpr float kL2Eps = 1e-6f;

// LPV = K / 8 lanes own one (token, head) vector of K elements, eight consecutive elements (16 bytes of bf16) each, so
// that every lane of a warp moves data for K = 64 ... 256; K = 512 takes two passes per lane (NV = 2).
// blockIdx.y = 0 for q, 1 for k.
template <int LPV>
__device__ __forceinline__ float group_sum(float v) {
#pragma unroll
  for (int o = LPV / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

template <typename T, int LPV, int NV>
__global__ void __launch_bounds__(256) l2norm_fwd_kernel(const b200gdn_prep_args a) {
  constexpr int VPW = 32 / LPV;   // vectors per warp
  const int lane = threadIdx.x & 31, sub = lane % LPV;
  const int64_t nvec = (int64_t)a.rows * a.H;
  const int64_t vec = ((int64_t)blockIdx.x * 8 + (threadIdx.x >> 5)) * VPW + lane / LPV;
  const bool live = vec < nvec;
  const void* src = blockIdx.y ? a.k : a.q;
  void* dst = blockIdx.y ? a.kn : a.qn;
  float* rstd = blockIdx.y ? a.rstd_k : a.rstd_q;
  float x[NV][8];
  float ss = 0.f;
#pragma unroll
  for (int v = 0; v < NV; ++v) {
    if (live) {
      load8<T>(src, vec * a.K + (v * LPV + sub) * 8, x[v]);
#pragma unroll
      for (int i = 0; i < 8; ++i) ss += x[v][i] * x[v][i];
    }
  }
  ss = group_sum<LPV>(ss);
  const float r = 1.f / sqrtf(ss + kL2Eps);
  if (live && sub == 0) rstd[vec] = r;
#pragma unroll
  for (int v = 0; v < NV; ++v) {
    if (live) {
#pragma unroll
      for (int i = 0; i < 8; ++i) x[v][i] *= r;
      store8<__nv_bfloat16>(dst, vec * a.K + (v * LPV + sub) * 8, x[v]);
    }
  }
}

// dx = (dy - (sum dy y) y) rstd with y = x rstd recomputed in fp32
template <typename T, int LPV, int NV>
__global__ void __launch_bounds__(256) l2norm_bwd_kernel(const b200gdn_prep_args a) {
  constexpr int VPW = 32 / LPV;
  const int lane = threadIdx.x & 31, sub = lane % LPV;
  const int64_t nvec = (int64_t)a.rows * a.H;
  const int64_t vec = ((int64_t)blockIdx.x * 8 + (threadIdx.x >> 5)) * VPW + lane / LPV;
  const bool live = vec < nvec;
  const void* src = blockIdx.y ? a.k : a.q;
  const void* dy = blockIdx.y ? a.dkn : a.dqn;
  void* dst = blockIdx.y ? a.dk : a.dq;
  const float r = live ? (blockIdx.y ? a.rstd_k : a.rstd_q)[vec] : 0.f;
  float y[NV][8], d[NV][8];
  float s = 0.f;
#pragma unroll
  for (int v = 0; v < NV; ++v) {
    if (live) {
      load8<T>(src, vec * a.K + (v * LPV + sub) * 8, y[v]);
      load8<__nv_bfloat16>(dy, vec * a.K + (v * LPV + sub) * 8, d[v]);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        y[v][i] *= r;
        s += d[v][i] * y[v][i];
      }
    }
  }
  s = group_sum<LPV>(s);
#pragma unroll
  for (int v = 0; v < NV; ++v) {
    if (live) {
#pragma unroll
      for (int i = 0; i < 8; ++i) d[v][i] = (d[v][i] - s * y[v][i]) * r;
      store8<T>(dst, vec * a.K + (v * LPV + sub) * 8, d[v]);
    }
  }
}

__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(expf(x)); }   // torch's threshold
__device__ __forceinline__ float sigmoid_f(float x) { return 1.f / (1.f + expf(-x)); }

template <typename T>
__global__ void __launch_bounds__(256) gate_beta_fwd_kernel(const b200gdn_prep_args a) {
  const int64_t n = (int64_t)a.rows * a.HV;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const int hv = (int)(i % a.HV);
    if (a.flags & B200GDN_PREP_GATE) {
      const float x = Io<T>::ld(a.g, i) + (a.dt_bias ? a.dt_bias[hv] : 0.f);
      a.g_out[i] = -expf(a.A_log[hv]) * softplus_f(x);
    }
    if (a.flags & B200GDN_PREP_BETA_SIGMOID) {
      const float s = (a.flags & B200GDN_PREP_NEG_EIGVAL) ? 2.f : 1.f;
      a.beta_out[i] = s * sigmoid_f(Io<T>::ld(a.beta, i));
    }
  }
}

// One CTA per B200GDN_PREP_PART_ROWS rows: thread (r, hv) walks rows r, r + RPB, ...; the per-head sums of
// dg g (-> dA_log) and dg_raw (-> ddt_bias) are reduced over the CTA in a fixed order and left as partials.
template <typename T>
__global__ void __launch_bounds__(256) gate_beta_bwd_kernel(const b200gdn_prep_args a) {
  extern __shared__ float red[];   // [2][256]
  const int HV = a.HV;
  const int rpb = 256 / HV;        // rows per pass (HV <= 256 checked by the host)
  const int hv = threadIdx.x % HV, r0 = threadIdx.x / HV;
  const int64_t row_beg = (int64_t)blockIdx.x * B200GDN_PREP_PART_ROWS;
  const int64_t row_end = min((int64_t)a.rows, row_beg + B200GDN_PREP_PART_ROWS);
  float sA = 0.f, sB = 0.f;
  if (r0 < rpb) {
    const float negA = (a.flags & B200GDN_PREP_GATE) ? -expf(a.A_log[hv]) : 0.f;
    const float bias = ((a.flags & B200GDN_PREP_GATE) && a.dt_bias) ? a.dt_bias[hv] : 0.f;
    const float s = (a.flags & B200GDN_PREP_NEG_EIGVAL) ? 2.f : 1.f;
    for (int64_t r = row_beg + r0; r < row_end; r += rpb) {
      const int64_t i = r * HV + hv;
      if (a.flags & B200GDN_PREP_GATE) {
        const float x = Io<T>::ld(a.g, i) + bias;
        const float dgi = a.dg[i];
        const float draw = dgi * negA * sigmoid_f(x);      // softplus' = sigmoid
        Io<T>::st(a.dg_raw, i, draw);
        sA += dgi * negA * softplus_f(x);                  // d/dA_log (-exp(A_log) sp) = the gate itself
        sB += draw;
      }
      if (a.flags & B200GDN_PREP_BETA_SIGMOID) {
        const float sg = sigmoid_f(Io<T>::ld(a.beta, i));
        Io<T>::st(a.dbeta_raw, i, a.dbeta[i] * s * sg * (1.f - sg));
      }
    }
  }
  if (a.flags & B200GDN_PREP_GATE) {
    red[threadIdx.x] = sA;
    red[256 + threadIdx.x] = sB;
    __syncthreads();
    if (threadIdx.x < HV) {
      float tA = 0.f, tB = 0.f;
      for (int r = 0; r < rpb; ++r) {
        tA += red[r * HV + threadIdx.x];
        tB += red[256 + r * HV + threadIdx.x];
      }
      a.partials[((int64_t)blockIdx.x * 2 + 0) * HV + threadIdx.x] = tA;
      a.partials[((int64_t)blockIdx.x * 2 + 1) * HV + threadIdx.x] = tB;
    }
  }
}

__global__ void gate_param_grad_kernel(const b200gdn_prep_args a, int n_part) {
  const int hv = blockIdx.x * blockDim.x + threadIdx.x;
  if (hv >= a.HV) return;
  float tA = 0.f, tB = 0.f;
  for (int p = 0; p < n_part; ++p) {
    tA += a.partials[((int64_t)p * 2 + 0) * a.HV + hv];
    tB += a.partials[((int64_t)p * 2 + 1) * a.HV + hv];
  }
  a.dA_log[hv] = tA;
  if (a.ddt_bias) a.ddt_bias[hv] = tB;
}

template <typename T, int LPV, int NV>
int launch_rows_k(const b200gdn_prep_args& a, cudaStream_t st, bool bwd) {
  const int64_t vecs = (int64_t)a.rows * a.H, per_cta = 8 * (32 / LPV);
  dim3 grid((unsigned)((vecs + per_cta - 1) / per_cta), 2);
  if (!bwd) {
    l2norm_fwd_kernel<T, LPV, NV><<<grid, 256, 0, st>>>(a);
    return check_launch("l2norm_fwd");
  }
  l2norm_bwd_kernel<T, LPV, NV><<<grid, 256, 0, st>>>(a);
  return check_launch("l2norm_bwd");
}

template <typename T>
int launch_rows(const b200gdn_prep_args& a, cudaStream_t st, bool bwd) {
  switch (a.K) {
    case 64: return launch_rows_k<T, 8, 1>(a, st, bwd);
    case 128: return launch_rows_k<T, 16, 1>(a, st, bwd);
    case 256: return launch_rows_k<T, 32, 1>(a, st, bwd);
    case 512: return launch_rows_k<T, 32, 2>(a, st, bwd);
  }
  return set_error(B200GDN_ERR_UNSUPPORTED, "l2norm: K=%d not built (64, 128, 256, 512 are)", a.K);
}

template <typename T>
int launch_vec(const b200gdn_prep_args& a, cudaStream_t st, bool bwd) {
  if (!bwd) {
    const int64_t n = (int64_t)a.rows * a.HV;
    const int64_t want = (n + 255) / 256;
    const int blocks = (int)(want < 148 * 8 ? want : 148 * 8);
    gate_beta_fwd_kernel<T><<<blocks, 256, 0, st>>>(a);
    return check_launch("gate_beta_fwd");
  }
  const int n_part = (a.rows + B200GDN_PREP_PART_ROWS - 1) / B200GDN_PREP_PART_ROWS;
  gate_beta_bwd_kernel<T><<<n_part, 256, 2 * 256 * sizeof(float), st>>>(a);
  if (int e = check_launch("gate_beta_bwd")) return e;
  if (a.flags & B200GDN_PREP_GATE) {
    gate_param_grad_kernel<<<(a.HV + 127) / 128, 128, 0, st>>>(a, n_part);
    return check_launch("gate_param_grad");
  }
  return 0;
}

}  // namespace

int launch_prep(const b200gdn_prep_args& a, cudaStream_t st, bool bwd) {
  if (a.flags & B200GDN_PREP_L2NORM) {
    int e = a.qk_dtype == 0 ? launch_rows<__nv_bfloat16>(a, st, bwd)
            : a.qk_dtype == 1 ? launch_rows<__half>(a, st, bwd)
                              : launch_rows<float>(a, st, bwd);
    if (e) return e;
  }
  if (a.flags & (B200GDN_PREP_GATE | B200GDN_PREP_BETA_SIGMOID)) {
    int e = a.gb_dtype == 0 ? launch_vec<__nv_bfloat16>(a, st, bwd)
            : a.gb_dtype == 1 ? launch_vec<__half>(a, st, bwd)
                              : launch_vec<float>(a, st, bwd);
    if (e) return e;
  }
  return 0;
}

}  // namespace gdn
