// Gated RMS norm over the head dimension, forward and backward: the step behind the mixer in fla.layers.GatedDeltaNet
// (fla/layers/gated_deltanet.py:355-357).  Replaces layer_norm_gated_fwd_kernel / layer_norm_gated_bwd_kernel of
// fla/modules/fused_norm_gate.py (36-124, 206-339) in their RMS form without residual:
//     rstd = 1 / sqrt(mean(x^2) + eps);   y = (x rstd weight + bias) act(g),   act(g) = g sigmoid(g) | sigmoid(g)
// Rows are (token, head) vectors of D = 64 .. 512 elements.  Pure HBM streaming: D / 8 lanes own a row, eight consecutive
// elements (16 bytes of bf16) each, so a warp covers 32 / (D / 8) rows per round with full-width accesses; persistent
// CTAs walk the rows with a grid stride and keep two rounds of loads in flight, so the backward pass can hold its
// dweight / dbias sums in registers and leave ONE partial row per CTA, which a second kernel adds in a fixed order
// (no atomics).
#include "gdn_common.cuh"
#include "rowio.cuh"

namespace gdn {
namespace {

constexpr int NT = 256;   // 8 warps

// sum over the LPV lanes that share a row (they differ in the low bits of the lane index)
template <int LPV>
__device__ __forceinline__ float row_sum(float v) {
#pragma unroll
  for (int o = LPV / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
// sum over the 32 / LPV lanes that hold the same columns of different rows
template <int LPV>
__device__ __forceinline__ float col_sum(float v) {
#pragma unroll
  for (int o = LPV; o < 32; o <<= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// LPV lanes per row, NV pieces of eight elements per lane: D = 8 LPV NV.  ROUNDS rounds of loads are in flight.
template <typename T, int LPV, int NV>
__global__ void __launch_bounds__(NT) norm_gate_fwd_kernel(const b200gdn_norm_gate_args a) {
  constexpr int D = 8 * LPV * NV, RW = 32 / LPV, ROUNDS = NV == 1 ? 2 : 1;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, sub = lane % LPV, rloc = lane / LPV;
  const bool sig = a.flags & B200GDN_NORM_GATE_SIGMOID;
  float w[NV][8], b[NV][8];
#pragma unroll
  for (int v = 0; v < NV; ++v)
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int d = (v * LPV + sub) * 8 + i;
      w[v][i] = a.weight ? a.weight[d] : 1.f;
      b[v][i] = a.bias ? a.bias[d] : 0.f;
    }
  const int64_t stride = (int64_t)gridDim.x * (NT / 32) * RW;
  // the loop bound is the warp's first row, so that every lane takes part in the shuffles of a round
  for (int64_t w0 = ((int64_t)blockIdx.x * (NT / 32) + warp) * RW; w0 < a.rows; w0 += ROUNDS * stride) {
    float x[ROUNDS][NV][8], g[ROUNDS][NV][8];
#pragma unroll
    for (int u = 0; u < ROUNDS; ++u) {
      const int64_t r = w0 + u * stride + rloc;
#pragma unroll
      for (int v = 0; v < NV; ++v) {
        if (r < a.rows) {
          load8<T>(a.x, r * D + (v * LPV + sub) * 8, x[u][v]);
          load8<T>(a.g, r * D + (v * LPV + sub) * 8, g[u][v]);
        } else {
#pragma unroll
          for (int i = 0; i < 8; ++i) { x[u][v][i] = 0.f; g[u][v][i] = 0.f; }
        }
      }
    }
#pragma unroll
    for (int u = 0; u < ROUNDS; ++u) {
      const int64_t r = w0 + u * stride + rloc;
      if (w0 + u * stride >= a.rows) break;   // warp-uniform
      float ss = 0.f;
#pragma unroll
      for (int v = 0; v < NV; ++v)
#pragma unroll
        for (int i = 0; i < 8; ++i) ss += x[u][v][i] * x[u][v][i];
      ss = row_sum<LPV>(ss);
      const float rstd = 1.f / sqrtf(ss / D + a.eps);
      if (r < a.rows) {
        if (sub == 0 && a.rstd != nullptr) a.rstd[r] = rstd;
#pragma unroll
        for (int v = 0; v < NV; ++v) {
          float y[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const float s = fast_sigmoid(g[u][v][i]);
            y[i] = (x[u][v][i] * rstd * w[v][i] + b[v][i]) * (sig ? s : g[u][v][i] * s);
          }
          store8<T>(a.y, r * D + (v * LPV + sub) * 8, y);
        }
      }
    }
  }
}

template <typename T, int LPV, int NV>
__global__ void __launch_bounds__(NT) norm_gate_bwd_kernel(const b200gdn_norm_gate_args a) {
  constexpr int D = 8 * LPV * NV, RW = 32 / LPV, ROUNDS = NV == 1 ? 2 : 1;
  __shared__ float part[2][NT / 32][D];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, sub = lane % LPV, rloc = lane / LPV;
  const bool sig = a.flags & B200GDN_NORM_GATE_SIGMOID;
  float w[NV][8], b[NV][8], dw[NV][8], db[NV][8];
#pragma unroll
  for (int v = 0; v < NV; ++v)
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int d = (v * LPV + sub) * 8 + i;
      w[v][i] = a.weight ? a.weight[d] : 1.f;
      b[v][i] = a.bias ? a.bias[d] : 0.f;
      dw[v][i] = 0.f;
      db[v][i] = 0.f;
    }
  const int64_t stride = (int64_t)gridDim.x * (NT / 32) * RW;
  for (int64_t w0 = ((int64_t)blockIdx.x * (NT / 32) + warp) * RW; w0 < a.rows; w0 += ROUNDS * stride) {
    float x[ROUNDS][NV][8], g[ROUNDS][NV][8], dy[ROUNDS][NV][8], rs[ROUNDS];
#pragma unroll
    for (int u = 0; u < ROUNDS; ++u) {
      const int64_t r = w0 + u * stride + rloc;
      rs[u] = r < a.rows ? a.rstd[r] : 0.f;
#pragma unroll
      for (int v = 0; v < NV; ++v) {
        if (r < a.rows) {
          load8<T>(a.x, r * D + (v * LPV + sub) * 8, x[u][v]);
          load8<T>(a.g, r * D + (v * LPV + sub) * 8, g[u][v]);
          load8<T>(a.dy, r * D + (v * LPV + sub) * 8, dy[u][v]);
        } else {   // a row past the end adds zeros to every sum
#pragma unroll
          for (int i = 0; i < 8; ++i) { x[u][v][i] = 0.f; g[u][v][i] = 0.f; dy[u][v][i] = 0.f; }
        }
      }
    }
#pragma unroll
    for (int u = 0; u < ROUNDS; ++u) {
      const int64_t r = w0 + u * stride + rloc;
      if (w0 + u * stride >= a.rows) break;   // warp-uniform
      const float rstd = rs[u];
      float dx[NV][8], dg[NV][8];
      float dot = 0.f;
#pragma unroll
      for (int v = 0; v < NV; ++v)
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float gi = g[u][v][i];
          const float s = fast_sigmoid(gi);
          const float act = sig ? s : gi * s;
          const float dact = sig ? s * (1.f - s) : s * (1.f + gi * (1.f - s));
          const float n = x[u][v][i] * rstd, y0 = n * w[v][i] + b[v][i];
          const float dy0 = dy[u][v][i] * act;
          dg[v][i] = dy[u][v][i] * y0 * dact;
          dw[v][i] += dy0 * n;
          db[v][i] += dy0;
          dx[v][i] = dy0 * w[v][i];   // gradient w.r.t. the normalised row
          dot += dx[v][i] * n;
        }
      dot = row_sum<LPV>(dot) / D;
      if (r < a.rows) {
#pragma unroll
        for (int v = 0; v < NV; ++v) {
#pragma unroll
          for (int i = 0; i < 8; ++i) dx[v][i] = rstd * (dx[v][i] - x[u][v][i] * rstd * dot);
          store8<T>(a.dx, r * D + (v * LPV + sub) * 8, dx[v]);
          store8<T>(a.dg, r * D + (v * LPV + sub) * 8, dg[v]);
        }
      }
    }
  }
  // one partial row per CTA: the rows of a warp added by shuffles, then the warps' sums in warp order
#pragma unroll
  for (int v = 0; v < NV; ++v)
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float sw = col_sum<LPV>(dw[v][i]), sb = col_sum<LPV>(db[v][i]);
      if (rloc == 0) {
        part[0][warp][(v * LPV + sub) * 8 + i] = sw;
        part[1][warp][(v * LPV + sub) * 8 + i] = sb;
      }
    }
  __syncthreads();
  for (int idx = threadIdx.x; idx < 2 * D; idx += NT) {
    const int which = idx / D, d = idx % D;
    float s = 0.f;
#pragma unroll
    for (int q = 0; q < NT / 32; ++q) s += part[which][q][d];
    a.partials[((int64_t)blockIdx.x * 2 + which) * D + d] = s;
  }
}

// dweight / dbias = sum of the CTAs' partial rows in a fixed order: warp q adds rows q, q + 32, ... for 32 consecutive
// outputs, then the 32 sums are added in warp order
constexpr int RW = 32;
__global__ void __launch_bounds__(32 * RW) norm_gate_param_reduce_kernel(const b200gdn_norm_gate_args a, int n_ctas) {
  __shared__ float part[RW][32];
  const int lane = threadIdx.x & 31, q = threadIdx.x >> 5;
  const int i = blockIdx.x * 32 + lane;   // D is a multiple of 32: every lane of a CTA has an output
  const int which = i / a.D, d = i % a.D;
  float s4[4] = {0.f, 0.f, 0.f, 0.f};   // four interleaved running sums, so that the loads overlap
  int c = q;
  for (; c + 3 * RW < n_ctas; c += 4 * RW) {
#pragma unroll
    for (int e = 0; e < 4; ++e) s4[e] += a.partials[((int64_t)(c + e * RW) * 2 + which) * a.D + d];
  }
  for (; c < n_ctas; c += RW) s4[0] += a.partials[((int64_t)c * 2 + which) * a.D + d];
  float s = (s4[0] + s4[1]) + (s4[2] + s4[3]);
  part[q][lane] = s;
  __syncthreads();
  if (q != 0) return;
#pragma unroll
  for (int r = 1; r < RW; ++r) s += part[r][lane];
  if (which == 0) { if (a.dweight) a.dweight[d] = s; }
  else if (a.dbias) a.dbias[d] = s;
}

template <typename T, int LPV, int NV>
int launch_t(const b200gdn_norm_gate_args& a, cudaStream_t st, bool bwd, int n_ctas) {
  if (!bwd) {
    norm_gate_fwd_kernel<T, LPV, NV><<<n_ctas, NT, 0, st>>>(a);
    return check_launch("norm_gate_fwd");
  }
  norm_gate_bwd_kernel<T, LPV, NV><<<n_ctas, NT, 0, st>>>(a);
  if (int e = check_launch("norm_gate_bwd")) return e;
  if (a.dweight != nullptr || a.dbias != nullptr) {
    norm_gate_param_reduce_kernel<<<2 * a.D / 32, 32 * RW, 0, st>>>(a, n_ctas);
    return check_launch("norm_gate_param_reduce");
  }
  return 0;
}

template <typename T>
int launch_d(const b200gdn_norm_gate_args& a, cudaStream_t st, bool bwd, int n_ctas) {
  switch (a.D) {
    case 64: return launch_t<T, 8, 1>(a, st, bwd, n_ctas);
    case 128: return launch_t<T, 16, 1>(a, st, bwd, n_ctas);
    case 256: return launch_t<T, 32, 1>(a, st, bwd, n_ctas);
    case 512: return launch_t<T, 32, 2>(a, st, bwd, n_ctas);
  }
  return set_error(B200GDN_ERR_UNSUPPORTED, "norm_gate: D=%d (64, 128, 256 and 512 are built)", a.D);
}

}  // namespace

// CTAs of the backward kernel for a row count: it leaves one partial row per CTA, so few CTAs that each walk many
// rows (at most 4 on each of 148 SMs)
int norm_gate_grid(int64_t rows) {
  const int64_t want = (rows + NT / 32 - 1) / (NT / 32);
  return (int)(want < 1 ? 1 : (want > 592 ? 592 : want));
}

int launch_norm_gate(const b200gdn_norm_gate_args& a, cudaStream_t st, bool bwd) {
  int n = norm_gate_grid(a.rows);
  if (!bwd) {   // the forward pass keeps nothing per CTA: more, shorter CTAs fill the SMs more evenly
    const int64_t want = (a.rows + NT / 32 - 1) / (NT / 32);
    n = (int)(want < 1 ? 1 : (want > 2368 ? 2368 : want));
  }
  return a.dtype == 0 ? launch_d<__nv_bfloat16>(a, st, bwd, n) : a.dtype == 1 ? launch_d<__half>(a, st, bwd, n) : launch_d<float>(a, st, bwd, n);
}

}  // namespace gdn
