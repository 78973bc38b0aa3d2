// Short causal depthwise convolution (+ SiLU) over token-major [rows, D] activations, forward and backward: the step
// in front of the mixer in fla.layers.GatedDeltaNet (fla/layers/gated_deltanet.py:247-300).  Replaces
// causal_conv1d_fwd_kernel / causal_conv1d_bwd_kernel (fla/modules/conv/triton/ops.py) for kernel sizes 2..4:
//     y[t, d] = act( bias[d] + sum_{w < W} weight[d, w] x[t - (W-1) + w, d] ) (+ residual[t, d])
// inside each sequence; inputs before the sequence start come from the cache initial_state[n, d, W - k] = x[-k]
// (k = 1..W-1) or are zero; final_state[n, d, :] holds the last W inputs of the sequence (cache entries shifted in when
// the sequence is shorter than W).
//
// Pure HBM streaming: a thread owns four consecutive channels (one 8-byte access per token for bf16) and walks 32
// consecutive tokens of one sequence (half a tile of the mixer's chunk table) with the W-1 previous inputs in
// registers, so x is read once (plus W-1 rows of overlap per share) and y written once.  The rows reach the thread
// through a private ring of asynchronous 8- or 16-byte copies in shared memory (sixteen tokens, twelve of them in flight
// while four are consumed): the DRAM latency is paid once per share, not once per round of loads, and the registers
// hold no look-ahead.  The backward pass recomputes the pre-activation, forms dx with a register ring over the W taps
// (the W-1 tokens after the share are re-evaluated for their contribution to its dx), writes the gradient of the
// cache for a sequence's first share, and leaves per-share partial sums of dweight / dbias that a second kernel adds
// in a fixed order (no atomics: results are bit-reproducible).
#include <type_traits>

#include "gdn_common.cuh"
#include "rowio.cuh"

namespace gdn {
namespace {

constexpr int CT = 64;    // threads per CTA: 512 channels
constexpr int SUB = 32;   // tokens per CTA: a 64-token tile is walked by two CTAs (blockIdx.z)
constexpr int NSUB = 64 / SUB;
constexpr int GRP = 4;    // tokens per copy group
constexpr int NGRP = 4;   // copy groups in the ring: three in flight, one being consumed
constexpr int RING = GRP * NGRP;

__device__ __forceinline__ float silu_f(float x) { return x * fast_sigmoid(x); }
__device__ __forceinline__ float dsilu_f(float x) {
  const float s = fast_sigmoid(x);
  return s * (1.f + x * (1.f - s));
}

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(smem_u32(smem)), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async8(void* smem, const void* gmem) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 8;\n" ::"r"(smem_u32(smem)), "l"(gmem) : "memory");
}

// A thread's ring of rows in shared memory: slot s holds the thread's C channels of one token as PIECES pieces of
// PB = 8 or 16 bytes, laid out [slot][piece][thread] so that the threads of a warp touch consecutive words.
template <typename T, int C>
struct RowRing {
  static constexpr int BYTES = C * (int)sizeof(T);            // 8, 16 or 32
  static constexpr int PB = BYTES < 16 ? BYTES : 16;
  static constexpr int PIECES = BYTES / PB;
  static constexpr size_t bytes = (size_t)RING * PIECES * CT * PB;
  unsigned char* base;   // this thread's word of slot 0, piece 0
  __device__ __forceinline__ unsigned char* word(int slot, int piece) const { return base + (size_t)(slot * PIECES + piece) * CT * PB; }
  __device__ __forceinline__ void fetch(int slot, const void* src, int64_t idx) const {
    const unsigned char* p = reinterpret_cast<const unsigned char*>(static_cast<const T*>(src) + idx);
#pragma unroll
    for (int h = 0; h < PIECES; ++h) {
      if constexpr (PB == 16) cp_async16(word(slot, h), p + h * 16);
      else cp_async8(word(slot, h), p);
    }
  }
  __device__ __forceinline__ void read(int slot, float (&x)[C]) const {
    if constexpr (BYTES == 8) {
      const uint2 u = *reinterpret_cast<const uint2*>(word(slot, 0));
      float y[8];
      unpack8<T>(make_uint4(u.x, u.y, 0u, 0u), y);
#pragma unroll
      for (int i = 0; i < 4; ++i) x[i] = y[i];
    } else if constexpr (sizeof(T) == 2) {
      unpack8<T>(*reinterpret_cast<const uint4*>(word(slot, 0)), x);
    } else {
#pragma unroll
      for (int h = 0; h < PIECES; ++h) {
        const uint4 u = *reinterpret_cast<const uint4*>(word(slot, h));
        x[4 * h] = __uint_as_float(u.x); x[4 * h + 1] = __uint_as_float(u.y);
        x[4 * h + 2] = __uint_as_float(u.z); x[4 * h + 3] = __uint_as_float(u.w);
      }
    }
  }
};

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

// the W inputs before token `row` of sequence n for channels d0..d0+C-1: hist[W-1] is x[row-1]; from the rows of x for a
// later tile, from the cache (or zeros) for a sequence's first tile
template <typename T, int W, int C>
__device__ __forceinline__ void load_history(const b200gdn_conv_args& a, const TileInfo& ti, int d0, float (&hist)[W][C]) {
#pragma unroll
  for (int k = 1; k <= W; ++k) {
    float (&h)[C] = hist[W - k];
    if (!ti.first) {
      load_c<T, C>(a.x, (int64_t)(ti.row - k) * a.D + d0, h);
    } else if (a.initial_state != nullptr && k < W) {
#pragma unroll
      for (int c = 0; c < C; ++c) h[c] = Io<T>::ld(a.initial_state, ((int64_t)ti.n * a.D + d0 + c) * W + (W - k));
    } else if (a.initial_state != nullptr) {   // k == W: the cache's oldest entry (only ever copied into the final state)
#pragma unroll
      for (int c = 0; c < C; ++c) h[c] = Io<T>::ld(a.initial_state, ((int64_t)ti.n * a.D + d0 + c) * W);
    } else {
#pragma unroll
      for (int c = 0; c < C; ++c) h[c] = 0.f;
    }
  }
}

template <typename T, int W, int C>
__global__ void __launch_bounds__(CT) conv_fwd_kernel(const b200gdn_conv_args a) {
  extern __shared__ __align__(16) unsigned char ring_mem[];
  const int d0 = (blockIdx.y * CT + threadIdx.x) * C;
  if (d0 >= a.D) return;   // no barrier below: every thread works on its own slots only
  const TileInfo ti = load_tile(a, blockIdx.x, blockIdx.z);
  if (ti.len <= 0) return;
  const RowRing<T, C> rx{ring_mem + threadIdx.x * RowRing<T, C>::PB};
  auto issue = [&](int gi) {   // one group: tokens 4 gi .. 4 gi + 3 of the share (an empty group past its end)
#pragma unroll
    for (int u = 0; u < GRP; ++u) {
      const int t = gi * GRP + u;
      if (t < ti.len) rx.fetch(t % RING, a.x, (int64_t)(ti.row + t) * a.D + d0);
    }
    cp_async_commit();
  };
#pragma unroll
  for (int gi = 0; gi < NGRP - 1; ++gi) issue(gi);
  const bool act = a.flags & B200GDN_CONV_SILU;
  float w[W][C], b[C], hist[W][C];
#pragma unroll
  for (int c = 0; c < C; ++c) {
#pragma unroll
    for (int j = 0; j < W; ++j) w[j][c] = a.weight[(int64_t)(d0 + c) * W + j];
    b[c] = a.bias ? a.bias[d0 + c] : 0.f;
  }
  load_history<T, W, C>(a, ti, d0, hist);
  // one token; FULL: the token is known to lie inside the share, so nothing in the body is conditional and the
  // compiler renames the history registers across the unrolled tokens of a group instead of moving them
  auto token = [&](int t, auto full) {
    if (!decltype(full)::value && t >= ti.len) return;
    float cur[C], y[C];
    rx.read(t % RING, cur);
#pragma unroll
    for (int c = 0; c < C; ++c) {
      float acc = b[c] + w[W - 1][c] * cur[c];
#pragma unroll
      for (int j = 0; j < W - 1; ++j) acc += w[j][c] * hist[j + 1][c];
      y[c] = act ? silu_f(acc) : acc;
    }
    const int64_t off = (int64_t)(ti.row + t) * a.D + d0;
    if (a.residual) {
      float r[C];
      load_c<T, C>(a.residual, off, r);
#pragma unroll
      for (int c = 0; c < C; ++c) y[c] += r[c];
    }
    store_c<T, C>(a.y, off, y);
#pragma unroll
    for (int j = 0; j < W - 1; ++j)
#pragma unroll
      for (int c = 0; c < C; ++c) hist[j][c] = hist[j + 1][c];
#pragma unroll
    for (int c = 0; c < C; ++c) hist[W - 1][c] = cur[c];
  };
  const int n_grp = (ti.len + GRP - 1) / GRP;
  for (int gi = 0; gi < n_grp; ++gi) {
    issue(gi + NGRP - 1);          // into the slots the previous round has consumed
    cp_async_wait<NGRP - 1>();     // all but the youngest three groups have landed: group gi is there
    if ((gi + 1) * GRP <= ti.len) {
#pragma unroll
      for (int u = 0; u < GRP; ++u) token(gi * GRP + u, std::true_type{});
    } else {
#pragma unroll
      for (int u = 0; u < GRP; ++u) token(gi * GRP + u, std::false_type{});
    }
  }
  cp_async_wait<0>();
  if (a.final_state != nullptr && ti.last) {
#pragma unroll
    for (int j = 0; j < W; ++j)
#pragma unroll
      for (int c = 0; c < C; ++c) Io<T>::st(a.final_state, ((int64_t)ti.n * a.D + d0 + c) * W + j, hist[j][c]);
  }
}

template <typename T, int W, int C>
__global__ void __launch_bounds__(CT) conv_bwd_kernel(const b200gdn_conv_args a) {
  extern __shared__ __align__(16) unsigned char ring_mem[];
  const int d0 = (blockIdx.y * CT + threadIdx.x) * C;
  if (d0 >= a.D) return;   // no barrier below: every thread works on its own slots only
  const int tile = blockIdx.x;
  const TileInfo ti = load_tile(a, tile, blockIdx.z);
  const bool act = a.flags & B200GDN_CONV_SILU;
  float* const part = a.partials ? a.partials + (((int64_t)tile * NSUB + blockIdx.z) * a.D + d0) * (W + 1) : nullptr;
  if (ti.len <= 0) {   // no token in this share: its partial sums are zeros
    if (part != nullptr)
      for (int i = 0; i < C * (W + 1); ++i) part[i] = 0.f;
    return;
  }
  // tokens of the same sequence after this share whose pre-activation gradient reaches its dx
  const int nxt = ti.after < W - 1 ? ti.after : W - 1;
  const int n_tok = ti.len + nxt;
  const RowRing<T, C> rx{ring_mem + threadIdx.x * RowRing<T, C>::PB}, rdy{ring_mem + RowRing<T, C>::bytes + threadIdx.x * RowRing<T, C>::PB};
  auto issue = [&](int gi) {
#pragma unroll
    for (int u = 0; u < GRP; ++u) {
      const int t = gi * GRP + u;
      if (t < n_tok) {
        const int64_t off = (int64_t)(ti.row + t) * a.D + d0;
        rx.fetch(t % RING, a.x, off);
        rdy.fetch(t % RING, a.dy, off);
      }
    }
    cp_async_commit();
  };
#pragma unroll
  for (int gi = 0; gi < NGRP - 1; ++gi) issue(gi);
  float w[W][C], b[C], hist[W][C];
#pragma unroll
  for (int c = 0; c < C; ++c) {
#pragma unroll
    for (int j = 0; j < W; ++j) w[j][c] = a.weight[(int64_t)(d0 + c) * W + j];
    b[c] = a.bias ? a.bias[d0 + c] : 0.f;
  }
  load_history<T, W, C>(a, ti, d0, hist);
  float ring[W][C];   // ring[k]: dx of token (u - k) so far, u the token being processed
  float dw[W][C], db[C];
#pragma unroll
  for (int j = 0; j < W; ++j)
#pragma unroll
    for (int c = 0; c < C; ++c) { ring[j][c] = 0.f; dw[j][c] = 0.f; }
#pragma unroll
  for (int c = 0; c < C; ++c) db[c] = 0.f;
  const int lo = (ti.first && a.dinitial_state != nullptr) ? -(W - 1) : 0;   // first token whose dx this share emits
  const int last = n_tok - 1 + (W - 1);   // the extra steps only flush the ring
  // one step; FULL: the token is known to lie inside the share (it is loaded, counted for the parameters, and no
  // step of its group is past the end), so only the store is conditional and the compiler renames the history and
  // ring registers across the unrolled steps of a group instead of moving them
  auto step = [&](int u, auto full) {
    constexpr bool FULL = decltype(full)::value;
    if (!FULL && u > last) return;
    float dpre[C];
    if (FULL || u < n_tok) {
      float cur[C], dy[C];
      rx.read(u % RING, cur);
      rdy.read(u % RING, dy);
#pragma unroll
      for (int c = 0; c < C; ++c) {
        float acc = b[c] + w[W - 1][c] * cur[c];
#pragma unroll
        for (int j = 0; j < W - 1; ++j) acc += w[j][c] * hist[j + 1][c];
        dpre[c] = act ? dy[c] * dsilu_f(acc) : dy[c];
      }
      if (FULL || u < ti.len) {   // the parameters' gradients: every token is counted by the share that owns it
#pragma unroll
        for (int c = 0; c < C; ++c) {
          db[c] += dpre[c];
          dw[W - 1][c] += dpre[c] * cur[c];
#pragma unroll
          for (int j = 0; j < W - 1; ++j) dw[j][c] += dpre[c] * hist[j + 1][c];
        }
      }
#pragma unroll
      for (int j = 0; j < W - 1; ++j)
#pragma unroll
        for (int c = 0; c < C; ++c) hist[j][c] = hist[j + 1][c];
#pragma unroll
      for (int c = 0; c < C; ++c) hist[W - 1][c] = cur[c];
    } else {
#pragma unroll
      for (int c = 0; c < C; ++c) dpre[c] = 0.f;
    }
    // dpre[u] reaches token u - k through tap W - 1 - k
#pragma unroll
    for (int k = 0; k < W; ++k)
#pragma unroll
      for (int c = 0; c < C; ++c) ring[k][c] += w[W - 1 - k][c] * dpre[c];
    const int s = u - (W - 1);   // this token has now received every contribution
    if (s >= lo && s < ti.len) {
      if (s >= 0) {
        store_c<T, C>(a.dx, (int64_t)(ti.row + s) * a.D + d0, ring[W - 1]);
      } else {   // an input before the sequence start: gradient of the cache entry x[s] = initial_state[n, d, W + s]
#pragma unroll
        for (int c = 0; c < C; ++c) Io<T>::st(a.dinitial_state, ((int64_t)ti.n * a.D + d0 + c) * W + (W + s), ring[W - 1][c]);
      }
    }
#pragma unroll
    for (int k = W - 1; k > 0; --k)
#pragma unroll
      for (int c = 0; c < C; ++c) ring[k][c] = ring[k - 1][c];
#pragma unroll
    for (int c = 0; c < C; ++c) ring[0][c] = 0.f;
  };
  for (int gi = 0; gi * GRP <= last; ++gi) {
    issue(gi + NGRP - 1);          // into the slots the previous round has consumed
    cp_async_wait<NGRP - 1>();     // group gi is there
    if ((gi + 1) * GRP <= ti.len) {
#pragma unroll
      for (int v = 0; v < GRP; ++v) step(gi * GRP + v, std::true_type{});
    } else {
#pragma unroll
      for (int v = 0; v < GRP; ++v) step(gi * GRP + v, std::false_type{});
    }
  }
  cp_async_wait<0>();
  if (ti.first && a.dinitial_state != nullptr) {   // the cache's oldest entry never enters the convolution
#pragma unroll
    for (int c = 0; c < C; ++c) Io<T>::st(a.dinitial_state, ((int64_t)ti.n * a.D + d0 + c) * W, 0.f);
  }
  if (part != nullptr) {
    float* p = part;
#pragma unroll
    for (int c = 0; c < C; ++c) {
#pragma unroll
      for (int j = 0; j < W; ++j) p[c * (W + 1) + j] = dw[j][c];
      p[c * (W + 1) + W] = db[c];
    }
  }
}

// dweight[d, w] / dbias[d] = sum over the shares in a fixed order: warp q of a CTA adds shares q, q + 16, ... for 32
// consecutive outputs (four interleaved running sums, so that the loads overlap), then the sixteen sums are added in
// warp order
constexpr int RW = 16;
__global__ void __launch_bounds__(32 * RW) conv_param_reduce_kernel(const b200gdn_conv_args a) {
  __shared__ float part[RW][32];
  const int lane = threadIdx.x & 31, q = threadIdx.x >> 5;
  const int64_t per_tile = (int64_t)a.D * (a.W + 1);
  const int64_t i = (int64_t)blockIdx.x * 32 + lane;
  float s4[4] = {0.f, 0.f, 0.f, 0.f};
  if (i < per_tile) {
    const int n = a.n_tiles * NSUB;
    int t = q;
    for (; t + 3 * RW < n; t += 4 * RW) {
#pragma unroll
      for (int e = 0; e < 4; ++e) s4[e] += a.partials[(int64_t)(t + e * RW) * per_tile + i];
    }
    for (; t < n; t += RW) s4[0] += a.partials[(int64_t)t * per_tile + i];
  }
  float s = (s4[0] + s4[1]) + (s4[2] + s4[3]);
  part[q][lane] = s;
  __syncthreads();
  if (q != 0 || i >= per_tile) return;
#pragma unroll
  for (int r = 1; r < RW; ++r) s += part[r][lane];
  const int d = (int)(i / (a.W + 1)), j = (int)(i % (a.W + 1));
  if (j < a.W) a.dweight[(int64_t)d * a.W + j] = s;
  else if (a.dbias != nullptr) a.dbias[d] = s;
}

// channels per thread: four in both passes.  With eight (16-byte accesses for bf16) the per-channel state of the backward
// pass (taps, history, dx ring, parameter sums) caps the SM at eight warps, and the forward pass at sixteen; the kernels
// are bound by instruction issue and dependent chains, not by access width, so the extra warps win (measured).
constexpr int C_FWD = 4, C_BWD = 4;

template <typename T, int W>
int launch_t(const b200gdn_conv_args& a, cudaStream_t st, bool bwd) {
  if (!bwd) {
    dim3 grid(a.n_tiles, (a.D / C_FWD + CT - 1) / CT, NSUB);
    constexpr size_t smem = RowRing<T, C_FWD>::bytes;
    if (int e = ensure_smem(conv_fwd_kernel<T, W, C_FWD>, smem)) return e;
    conv_fwd_kernel<T, W, C_FWD><<<grid, CT, smem, st>>>(a);
    return check_launch("conv_fwd");
  }
  dim3 grid(a.n_tiles, (a.D / C_BWD + CT - 1) / CT, NSUB);
  constexpr size_t smem = 2 * RowRing<T, C_BWD>::bytes;
  if (int e = ensure_smem(conv_bwd_kernel<T, W, C_BWD>, smem)) return e;
  conv_bwd_kernel<T, W, C_BWD><<<grid, CT, smem, st>>>(a);
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
