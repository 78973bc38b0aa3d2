// Gated RMS norm over the head dimension, forward and backward: the step behind the mixer in fla.layers.GatedDeltaNet
// (fla/layers/gated_deltanet.py:355-357).  Replaces layer_norm_gated_fwd_kernel / layer_norm_gated_bwd_kernel of
// fla/modules/fused_norm_gate.py (36-124, 206-339) in their RMS form without residual:
//     rstd = 1 / sqrt(mean(x^2) + eps);   y = (x rstd weight + bias) act(g),   act(g) = g sigmoid(g) | sigmoid(g)
// Rows are (token, head) vectors of D = 64 .. 512 elements.  Pure HBM streaming: one warp owns a row, a lane D / 32
// consecutive elements (8 or 16 bytes per access at D = 128); persistent CTAs walk the rows with a grid stride, so the
// backward pass can keep its dweight / dbias sums in registers and leave ONE partial row per CTA, which a second kernel
// adds in a fixed order (no atomics).
#include "gdn_common.cuh"
#include "rowio.cuh"

namespace gdn {
namespace {

constexpr int NT = 256;   // 8 warps

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// VPT consecutive elements of a row with the widest access their size allows (16, 8 or 4 bytes)
template <typename T, int VPT>
__device__ __forceinline__ void load_row(const void* base, int64_t idx, float (&x)[VPT]) {
  constexpr int BYTES = VPT * (int)sizeof(T);
  alignas(16) unsigned char buf[BYTES];
  const unsigned char* src = static_cast<const unsigned char*>(base) + idx * (int64_t)sizeof(T);
  if constexpr (BYTES % 16 == 0) {
#pragma unroll
    for (int i = 0; i < BYTES / 16; ++i) reinterpret_cast<uint4*>(buf)[i] = reinterpret_cast<const uint4*>(src)[i];
  } else if constexpr (BYTES == 8) {
    *reinterpret_cast<uint2*>(buf) = *reinterpret_cast<const uint2*>(src);
  } else {
    static_assert(BYTES == 4, "row slice of 4, 8 or a multiple of 16 bytes");
    *reinterpret_cast<uint32_t*>(buf) = *reinterpret_cast<const uint32_t*>(src);
  }
#pragma unroll
  for (int i = 0; i < VPT; ++i) x[i] = Io<T>::ld(buf, i);
}
template <typename T, int VPT>
__device__ __forceinline__ void store_row(void* base, int64_t idx, const float (&x)[VPT]) {
  constexpr int BYTES = VPT * (int)sizeof(T);
  alignas(16) unsigned char buf[BYTES];
#pragma unroll
  for (int i = 0; i < VPT; ++i) Io<T>::st(buf, i, x[i]);
  unsigned char* dst = static_cast<unsigned char*>(base) + idx * (int64_t)sizeof(T);
  if constexpr (BYTES % 16 == 0) {
#pragma unroll
    for (int i = 0; i < BYTES / 16; ++i) reinterpret_cast<uint4*>(dst)[i] = reinterpret_cast<const uint4*>(buf)[i];
  } else if constexpr (BYTES == 8) {
    *reinterpret_cast<uint2*>(dst) = *reinterpret_cast<const uint2*>(buf);
  } else {
    *reinterpret_cast<uint32_t*>(dst) = *reinterpret_cast<const uint32_t*>(buf);
  }
}

template <typename T, int VPT>
__global__ void __launch_bounds__(NT) norm_gate_fwd_kernel(const b200gdn_norm_gate_args a) {
  constexpr int D = VPT * 32;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const bool sig = a.flags & B200GDN_NORM_GATE_SIGMOID;
  float w[VPT], b[VPT];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    w[i] = a.weight ? a.weight[lane * VPT + i] : 1.f;
    b[i] = a.bias ? a.bias[lane * VPT + i] : 0.f;
  }
  for (int64_t r = (int64_t)blockIdx.x * (NT / 32) + warp; r < a.rows; r += (int64_t)gridDim.x * (NT / 32)) {
    const int64_t off = r * D + lane * VPT;
    float x[VPT], g[VPT], y[VPT];
    load_row<T, VPT>(a.x, off, x);
    load_row<T, VPT>(a.g, off, g);
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) ss += x[i] * x[i];
    ss = warp_sum(ss);
    const float rstd = 1.f / sqrtf(ss / D + a.eps);
    if (lane == 0 && a.rstd != nullptr) a.rstd[r] = rstd;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const float s = __fdividef(1.f, 1.f + __expf(-g[i]));   // approximate reciprocal: one MUFU op instead of the IEEE division
      y[i] = (x[i] * rstd * w[i] + b[i]) * (sig ? s : g[i] * s);
    }
    store_row<T, VPT>(a.y, off, y);
  }
}

template <typename T, int VPT>
__global__ void __launch_bounds__(NT) norm_gate_bwd_kernel(const b200gdn_norm_gate_args a) {
  constexpr int D = VPT * 32;
  __shared__ float part[2][NT / 32][D];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const bool sig = a.flags & B200GDN_NORM_GATE_SIGMOID;
  float w[VPT], b[VPT], dw[VPT], db[VPT];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    w[i] = a.weight ? a.weight[lane * VPT + i] : 1.f;
    b[i] = a.bias ? a.bias[lane * VPT + i] : 0.f;
    dw[i] = 0.f;
    db[i] = 0.f;
  }
  for (int64_t r = (int64_t)blockIdx.x * (NT / 32) + warp; r < a.rows; r += (int64_t)gridDim.x * (NT / 32)) {
    const int64_t off = r * D + lane * VPT;
    float x[VPT], g[VPT], dy[VPT], dx[VPT], dg[VPT];
    load_row<T, VPT>(a.x, off, x);
    load_row<T, VPT>(a.g, off, g);
    load_row<T, VPT>(a.dy, off, dy);
    const float rstd = a.rstd[r];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const float s = __fdividef(1.f, 1.f + __expf(-g[i]));
      const float act = sig ? s : g[i] * s;
      const float dact = sig ? s * (1.f - s) : s * (1.f + g[i] * (1.f - s));
      const float n = x[i] * rstd, y0 = n * w[i] + b[i];
      const float dy0 = dy[i] * act;
      dg[i] = dy[i] * y0 * dact;
      dw[i] += dy0 * n;
      db[i] += dy0;
      dx[i] = dy0 * w[i];   // gradient w.r.t. the normalised row
      dot += dx[i] * n;
    }
    dot = warp_sum(dot) / D;
#pragma unroll
    for (int i = 0; i < VPT; ++i) dx[i] = rstd * (dx[i] - x[i] * rstd * dot);
    store_row<T, VPT>(a.dx, off, dx);
    store_row<T, VPT>(a.dg, off, dg);
  }
  // one partial row per CTA: the warps' sums added in warp order
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    part[0][warp][lane * VPT + i] = dw[i];
    part[1][warp][lane * VPT + i] = db[i];
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
  float s = 0.f;
  for (int c = q; c < n_ctas; c += RW) s += a.partials[((int64_t)c * 2 + which) * a.D + d];
  part[q][lane] = s;
  __syncthreads();
  if (q != 0) return;
#pragma unroll
  for (int r = 1; r < RW; ++r) s += part[r][lane];
  if (which == 0) { if (a.dweight) a.dweight[d] = s; }
  else if (a.dbias) a.dbias[d] = s;
}

template <typename T, int VPT>
int launch_t(const b200gdn_norm_gate_args& a, cudaStream_t st, bool bwd, int n_ctas) {
  if (!bwd) {
    norm_gate_fwd_kernel<T, VPT><<<n_ctas, NT, 0, st>>>(a);
    return check_launch("norm_gate_fwd");
  }
  norm_gate_bwd_kernel<T, VPT><<<n_ctas, NT, 0, st>>>(a);
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
    case 64: return launch_t<T, 2>(a, st, bwd, n_ctas);
    case 128: return launch_t<T, 4>(a, st, bwd, n_ctas);
    case 256: return launch_t<T, 8>(a, st, bwd, n_ctas);
    case 512: return launch_t<T, 16>(a, st, bwd, n_ctas);
  }
  return set_error(B200GDN_ERR_UNSUPPORTED, "norm_gate: D=%d (64, 128, 256 and 512 are built)", a.D);
}

}  // namespace

// CTAs of the (persistent) norm kernels for a row count; the backward pass leaves one partial row per CTA
int norm_gate_grid(int64_t rows) {
  const int64_t want = (rows + NT / 32 - 1) / (NT / 32);
  return (int)(want < 1 ? 1 : (want > 1184 ? 1184 : want));   // at most 8 CTAs on each of 148 SMs
}

int launch_norm_gate(const b200gdn_norm_gate_args& a, cudaStream_t st, bool bwd) {
  const int n = norm_gate_grid(a.rows);
  return a.dtype == 0 ? launch_d<__nv_bfloat16>(a, st, bwd, n) : a.dtype == 1 ? launch_d<__half>(a, st, bwd, n) : launch_d<float>(a, st, bwd, n);
}

}  // namespace gdn
