// Short causal depthwise convolution (+ SiLU) over token-major [rows, D] activations, forward and backward: the step
// in front of the mixer in fla.layers.GatedDeltaNet (fla/layers/gated_deltanet.py:247-300).  Replaces
// causal_conv1d_fwd_kernel / causal_conv1d_bwd_kernel (fla/modules/conv/triton/ops.py) for kernel sizes 2..4:
//     y[t, d] = act( bias[d] + sum_{w < W} weight[d, w] x[t - (W-1) + w, d] ) (+ residual[t, d])
// inside each sequence; inputs before the sequence start come from the cache initial_state[n, d, W - k] = x[-k]
// (k = 1..W-1) or are zero; final_state[n, d, :] holds the last W inputs of the sequence (cache entries shifted in when
// the sequence is shorter than W).
//
// Pure HBM streaming: a thread owns eight consecutive channels (one 16-byte access per token for bf16) and walks the
// up-to-64 tokens of one tile of one sequence with the W-1 previous inputs in registers, so x is read once (plus W-1
// rows of overlap per tile) and y written once.  Tiles come from the same (sequence, first row, length, index) table
// as the mixer's chunks.  The backward pass recomputes the pre-activation, forms dx with a register ring over the
// W taps (the W-1 tokens after the tile are re-evaluated for their contribution to the tile's dx), writes the
// gradient of the cache for a sequence's first tile, and leaves per-tile partial sums of dweight / dbias that a
// second kernel adds in a fixed order (no atomics: results are bit-reproducible).
#include "gdn_common.cuh"
#include "rowio.cuh"

namespace gdn {
namespace {

constexpr int CT = 128;   // threads per CTA: 1024 channels
constexpr int SUB = 32;   // tokens per CTA: a 64-token tile is walked by two CTAs (blockIdx.z), for twice the loads in flight
constexpr int NSUB = 64 / SUB;

// approximate reciprocal (one MUFU op): the IEEE division costs more instructions than the rest of a tap
__device__ __forceinline__ float sigmoid_f(float x) { return __fdividef(1.f, 1.f + __expf(-x)); }
__device__ __forceinline__ float silu_f(float x) { return x * sigmoid_f(x); }
__device__ __forceinline__ float dsilu_f(float x) {
  const float s = sigmoid_f(x);
  return s * (1.f + x * (1.f - s));
}

// One CTA's share of a tile: `row` is its first token, `len` its token count, `first` / `last` say whether it starts /
// ends its sequence, `after` how many tokens of the sequence follow it (capped at 3, the largest overlap needed).
struct TileInfo {
  int n, row, len;
  bool first, last;
  int after;
};
__device__ __forceinline__ TileInfo load_tile(const b200gdn_conv_args& a, int tile, int sub) {
  const int4 m = reinterpret_cast<const int4*>(a.tile_meta)[tile];
  const int ntiles = a.seq_meta[2 * m.x + 1];
  const int start = sub * SUB;
  TileInfo ti;
  ti.n = m.x;
  ti.row = m.y + start;
  ti.len = m.z - start < SUB ? m.z - start : SUB;   // <= 0: nothing to do for this CTA
  ti.first = m.w == 0 && sub == 0;
  const int rest = m.z - start - ti.len;            // tokens of the tile behind this share
  ti.last = m.w == ntiles - 1 && rest <= 0;
  int after = rest;
  if (after < 3 && m.w < ntiles - 1) after += a.tile_meta[4 * (tile + 1) + 2];
  ti.after = after < 3 ? (after < 0 ? 0 : after) : 3;
  return ti;
}

// the W inputs before token `row` of sequence n for channels d0..d0+7: hist[W-1] is x[row-1]; from the rows of x for a
// later tile, from the cache (or zeros) for a sequence's first tile
template <typename T, int W>
__device__ __forceinline__ void load_history(const b200gdn_conv_args& a, const TileInfo& ti, int d0, float (&hist)[W][8]) {
#pragma unroll
  for (int k = 1; k <= W; ++k) {
    float (&h)[8] = hist[W - k];
    if (!ti.first) {
      load8<T>(a.x, (int64_t)(ti.row - k) * a.D + d0, h);
    } else if (a.initial_state != nullptr && k < W) {
#pragma unroll
      for (int c = 0; c < 8; ++c) h[c] = Io<T>::ld(a.initial_state, ((int64_t)ti.n * a.D + d0 + c) * W + (W - k));
    } else if (a.initial_state != nullptr) {   // k == W: the cache's oldest entry (only ever copied into the final state)
#pragma unroll
      for (int c = 0; c < 8; ++c) h[c] = Io<T>::ld(a.initial_state, ((int64_t)ti.n * a.D + d0 + c) * W);
    } else {
#pragma unroll
      for (int c = 0; c < 8; ++c) h[c] = 0.f;
    }
  }
}

template <typename T, int W>
__global__ void __launch_bounds__(CT) conv_fwd_kernel(const b200gdn_conv_args a) {
  const int d0 = (blockIdx.y * CT + threadIdx.x) * 8;
  if (d0 >= a.D) return;
  const TileInfo ti = load_tile(a, blockIdx.x, blockIdx.z);
  if (ti.len <= 0) return;
  const bool act = a.flags & B200GDN_CONV_SILU;
  float w[W][8], b[8], hist[W][8];
#pragma unroll
  for (int c = 0; c < 8; ++c) {
#pragma unroll
    for (int j = 0; j < W; ++j) w[j][c] = a.weight[(int64_t)(d0 + c) * W + j];
    b[c] = a.bias ? a.bias[d0 + c] : 0.f;
  }
  load_history<T, W>(a, ti, d0, hist);
  for (int t0 = 0; t0 < ti.len; t0 += 4) {
    // four tokens per round: their loads are issued together, the taps then walk them in order
    float cur[4][8], r[4][8];
#pragma unroll
    for (int u = 0; u < 4; ++u)
      if (t0 + u < ti.len) {
        const int64_t off = (int64_t)(ti.row + t0 + u) * a.D + d0;
        load8<T>(a.x, off, cur[u]);
        if (a.residual) load8<T>(a.residual, off, r[u]);
      }
#pragma unroll
    for (int u = 0; u < 4; ++u)
      if (t0 + u < ti.len) {
        float y[8];
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          float acc = b[c] + w[W - 1][c] * cur[u][c];
#pragma unroll
          for (int j = 0; j < W - 1; ++j) acc += w[j][c] * hist[j + 1][c];
          y[c] = act ? silu_f(acc) : acc;
          if (a.residual) y[c] += r[u][c];
        }
        store8<T>(a.y, (int64_t)(ti.row + t0 + u) * a.D + d0, y);
#pragma unroll
        for (int j = 0; j < W - 1; ++j)
#pragma unroll
          for (int c = 0; c < 8; ++c) hist[j][c] = hist[j + 1][c];
#pragma unroll
        for (int c = 0; c < 8; ++c) hist[W - 1][c] = cur[u][c];
      }
  }
  if (a.final_state != nullptr && ti.last) {
#pragma unroll
    for (int j = 0; j < W; ++j)
#pragma unroll
      for (int c = 0; c < 8; ++c) Io<T>::st(a.final_state, ((int64_t)ti.n * a.D + d0 + c) * W + j, hist[j][c]);
  }
}

template <typename T, int W>
__global__ void __launch_bounds__(CT) conv_bwd_kernel(const b200gdn_conv_args a) {
  const int d0 = (blockIdx.y * CT + threadIdx.x) * 8;
  if (d0 >= a.D) return;
  const int tile = blockIdx.x;
  const TileInfo ti = load_tile(a, tile, blockIdx.z);
  const bool act = a.flags & B200GDN_CONV_SILU;
  float* const part = a.partials ? a.partials + (((int64_t)tile * NSUB + blockIdx.z) * a.D + d0) * (W + 1) : nullptr;
  if (ti.len <= 0) {   // no token in this share: its partial sums are zeros
    if (part != nullptr)
      for (int i = 0; i < 8 * (W + 1); ++i) part[i] = 0.f;
    return;
  }
  // tokens of the same sequence after this share whose pre-activation gradient reaches its dx
  const int nxt = ti.after < W - 1 ? ti.after : W - 1;
  float w[W][8], b[8], hist[W][8];
#pragma unroll
  for (int c = 0; c < 8; ++c) {
#pragma unroll
    for (int j = 0; j < W; ++j) w[j][c] = a.weight[(int64_t)(d0 + c) * W + j];
    b[c] = a.bias ? a.bias[d0 + c] : 0.f;
  }
  load_history<T, W>(a, ti, d0, hist);
  float ring[W][8];   // ring[k]: dx of token (u - k) so far, u the token being processed
  float dw[W][8], db[8];
#pragma unroll
  for (int j = 0; j < W; ++j)
#pragma unroll
    for (int c = 0; c < 8; ++c) { ring[j][c] = 0.f; dw[j][c] = 0.f; }
#pragma unroll
  for (int c = 0; c < 8; ++c) db[c] = 0.f;
  const int lo = (ti.first && a.dinitial_state != nullptr) ? -(W - 1) : 0;   // first token whose dx this share emits
  const int last = ti.len + nxt - 1 + (W - 1);   // the extra steps only flush the ring
  for (int u0 = 0; u0 <= last; u0 += 4) {
    // four tokens per round: their loads are issued together
    float cx[4][8], cdy[4][8];
#pragma unroll
    for (int v = 0; v < 4; ++v)
      if (u0 + v < ti.len + nxt) {
        const int64_t off = (int64_t)(ti.row + u0 + v) * a.D + d0;
        load8<T>(a.x, off, cx[v]);
        load8<T>(a.dy, off, cdy[v]);
      }
#pragma unroll
    for (int v = 0; v < 4; ++v) {
      const int u = u0 + v;
      if (u > last) break;
      float dpre[8];
      if (u < ti.len + nxt) {
        const float (&cur)[8] = cx[v];
        const float (&dy)[8] = cdy[v];
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          float acc = b[c] + w[W - 1][c] * cur[c];
#pragma unroll
          for (int j = 0; j < W - 1; ++j) acc += w[j][c] * hist[j + 1][c];
          dpre[c] = act ? dy[c] * dsilu_f(acc) : dy[c];
        }
        if (u < ti.len) {   // the parameters' gradients: every token is counted by the share that owns it
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            db[c] += dpre[c];
            dw[W - 1][c] += dpre[c] * cur[c];
#pragma unroll
            for (int j = 0; j < W - 1; ++j) dw[j][c] += dpre[c] * hist[j + 1][c];
          }
        }
#pragma unroll
        for (int j = 0; j < W - 1; ++j)
#pragma unroll
          for (int c = 0; c < 8; ++c) hist[j][c] = hist[j + 1][c];
#pragma unroll
        for (int c = 0; c < 8; ++c) hist[W - 1][c] = cur[c];
      } else {
#pragma unroll
        for (int c = 0; c < 8; ++c) dpre[c] = 0.f;
      }
      // dpre[u] reaches token u - k through tap W - 1 - k
#pragma unroll
      for (int k = 0; k < W; ++k)
#pragma unroll
        for (int c = 0; c < 8; ++c) ring[k][c] += w[W - 1 - k][c] * dpre[c];
      const int s = u - (W - 1);   // this token has now received every contribution
      if (s >= lo && s < ti.len) {
        if (s >= 0) {
          store8<T>(a.dx, (int64_t)(ti.row + s) * a.D + d0, ring[W - 1]);
        } else {   // an input before the sequence start: gradient of the cache entry x[s] = initial_state[n, d, W + s]
#pragma unroll
          for (int c = 0; c < 8; ++c) Io<T>::st(a.dinitial_state, ((int64_t)ti.n * a.D + d0 + c) * W + (W + s), ring[W - 1][c]);
        }
      }
#pragma unroll
      for (int k = W - 1; k > 0; --k)
#pragma unroll
        for (int c = 0; c < 8; ++c) ring[k][c] = ring[k - 1][c];
#pragma unroll
      for (int c = 0; c < 8; ++c) ring[0][c] = 0.f;
    }
  }
  if (ti.first && a.dinitial_state != nullptr) {   // the cache's oldest entry never enters the convolution
#pragma unroll
    for (int c = 0; c < 8; ++c) Io<T>::st(a.dinitial_state, ((int64_t)ti.n * a.D + d0 + c) * W, 0.f);
  }
  if (part != nullptr) {
    float* p = part;
#pragma unroll
    for (int c = 0; c < 8; ++c) {
#pragma unroll
      for (int j = 0; j < W; ++j) p[c * (W + 1) + j] = dw[j][c];
      p[c * (W + 1) + W] = db[c];
    }
  }
}

// dweight[d, w] / dbias[d] = sum over the shares in a fixed order: warp q of a CTA adds shares q, q + 8, ... for 32
// consecutive outputs, then the eight sums are added in warp order
constexpr int RW = 8;
__global__ void __launch_bounds__(32 * RW) conv_param_reduce_kernel(const b200gdn_conv_args a) {
  __shared__ float part[RW][32];
  const int lane = threadIdx.x & 31, q = threadIdx.x >> 5;
  const int64_t per_tile = (int64_t)a.D * (a.W + 1);
  const int64_t i = (int64_t)blockIdx.x * 32 + lane;
  float s = 0.f;
  if (i < per_tile)
    for (int t = q; t < a.n_tiles * NSUB; t += RW) s += a.partials[(int64_t)t * per_tile + i];
  part[q][lane] = s;
  __syncthreads();
  if (q != 0 || i >= per_tile) return;
#pragma unroll
  for (int r = 1; r < RW; ++r) s += part[r][lane];
  const int d = (int)(i / (a.W + 1)), j = (int)(i % (a.W + 1));
  if (j < a.W) a.dweight[(int64_t)d * a.W + j] = s;
  else if (a.dbias != nullptr) a.dbias[d] = s;
}

template <typename T, int W>
int launch_t(const b200gdn_conv_args& a, cudaStream_t st, bool bwd) {
  dim3 grid(a.n_tiles, (a.D / 8 + CT - 1) / CT, NSUB);
  if (!bwd) {
    conv_fwd_kernel<T, W><<<grid, CT, 0, st>>>(a);
    return check_launch("conv_fwd");
  }
  conv_bwd_kernel<T, W><<<grid, CT, 0, st>>>(a);
  if (int e = check_launch("conv_bwd")) return e;
  if (a.partials != nullptr && a.dweight != nullptr) {
    const int64_t n = (int64_t)a.D * (a.W + 1);
    conv_param_reduce_kernel<<<(unsigned)((n + 31) / 32), 32 * RW, 0, st>>>(a);
    return check_launch("conv_param_reduce");
  }
  return 0;
}

template <typename T>
int launch_w(const b200gdn_conv_args& a, cudaStream_t st, bool bwd) {
  if (a.W == 4) return launch_t<T, 4>(a, st, bwd);
  if (a.W == 3) return launch_t<T, 3>(a, st, bwd);
  if (a.W == 2) return launch_t<T, 2>(a, st, bwd);
  return set_error(B200GDN_ERR_UNSUPPORTED, "conv: kernel size %d (2, 3 and 4 are built)", a.W);
}

}  // namespace

int launch_conv(const b200gdn_conv_args& a, cudaStream_t st, bool bwd) {
  return a.dtype == 0 ? launch_w<__nv_bfloat16>(a, st, bwd) : a.dtype == 1 ? launch_w<__half>(a, st, bwd) : launch_w<float>(a, st, bwd);
}

}  // namespace gdn
