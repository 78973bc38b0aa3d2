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
#include "tc5.cuh"
#include "tma.cuh"

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

// Slot of the state pool that sequence n uses.  With a pool (state_indices) and a known pool size, an index outside
// [0, n_slots) marks a padding sequence (serving engines use -1): it reads slot 0, its output is meaningless and its
// state is not written back (`*writeback` = false), so no access leaves the pool.
__device__ __forceinline__ int64_t state_slot(const b200gdn_recurrent_args& a, int n, bool* writeback) {
  *writeback = true;
  if (a.state_indices == nullptr) return n;
  const int64_t slot = a.state_indices[n];
  if (a.n_slots > 0 && (slot < 0 || slot >= a.n_slots)) {
    *writeback = false;
    return 0;
  }
  return slot;
}

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
  bool writeback;
  const int64_t slot = state_slot(a, n, &writeback);   // which state of the pool this sequence uses
  const float* h0 = a.h0 ? a.h0 + (slot * a.HV + hv) * DK * DV : nullptr;
  float* ht = (a.ht && writeback) ? a.ht + (slot * a.HV + hv) * DK * DV : nullptr;
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

// [K,V] layout with V = 128: one CTA of eight warps owns the whole state of one (sequence, head) - K rows of 512
// contiguous bytes, i.e. one contiguous block of K * 512 bytes - so that every DRAM page of the state is opened once
// for the read and once for the write (the 32-channel slices of the kernel above touch each page four times, which
// costs about a quarter of the bandwidth at large batch).  Warp w keeps rows [w K/8, (w+1) K/8), lane l the columns
// 4 l .. 4 l + 3: a warp moves one full row per 128-bit access.
template <int DK>
__global__ void __launch_bounds__(256, 2) recurrent_rows_kernel(const b200gdn_recurrent_args a) {
  constexpr int NT = 256, DV = 128, RW = DK / 8;   // rows per warp
  __shared__ __align__(16) float qs[DK];
  __shared__ __align__(16) float ks[DK];
  __shared__ __align__(16) float vs[DV];
  __shared__ __align__(16) float red[8][DV];
  __shared__ float sc[2];  // decay, beta

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int hv = blockIdx.x, n = blockIdx.y;
  const int G = a.HV / a.H, hq = hv / G;
  int64_t bos, len;
  if (a.cu_seqlens != nullptr) {
    bos = a.cu_seqlens[n];
    len = a.cu_seqlens[n + 1] - bos;
  } else {
    bos = (int64_t)n * a.T;
    len = a.T;
  }
  float4 st[RW];
  bool writeback;
  const int64_t slot = state_slot(a, n, &writeback);   // which state of the pool this sequence uses
  const float* h0 = a.h0 ? a.h0 + (slot * a.HV + hv) * DK * DV : nullptr;
  float* ht = (a.ht && writeback) ? a.ht + (slot * a.HV + hv) * DK * DV : nullptr;
  const int col = 4 * lane, r0 = warp * RW;
#pragma unroll
  for (int i = 0; i < RW; ++i)
    st[i] = h0 ? *reinterpret_cast<const float4*>(h0 + (int64_t)(r0 + i) * DV + col) : make_float4(0.f, 0.f, 0.f, 0.f);

  for (int64_t tok = 0; tok < len; ++tok) {
    const int64_t row = bos + tok;
    __syncthreads();  // previous token's shared inputs are no longer read
    if (tid < DK) {
      qs[tid] = ld_elem(a.q, (row * a.H + hq) * DK + tid, a.qkv_dtype);
      ks[tid] = ld_elem(a.k, (row * a.H + hq) * DK + tid, a.qkv_dtype);
    } else if (tid < DK + DV) {
      vs[tid - DK] = ld_elem(a.v, (row * a.HV + hv) * DV + tid - DK, a.qkv_dtype);
    }
    if (tid == NT - 1) {
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

    // S <- S decay;  partial S^T k over this warp's rows
    float4 d = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int i = 0; i < RW; ++i) {
      st[i].x *= decay; st[i].y *= decay; st[i].z *= decay; st[i].w *= decay;
      const float kk = ks[r0 + i] * kn;
      d.x += st[i].x * kk; d.y += st[i].y * kk; d.z += st[i].z * kk; d.w += st[i].w * kk;
    }
    *reinterpret_cast<float4*>(&red[warp][col]) = d;
    __syncthreads();
    float4 r;
    {
      float4 s = *reinterpret_cast<const float4*>(&red[0][col]);
#pragma unroll
      for (int w = 1; w < 8; ++w) {
        const float4 x = *reinterpret_cast<const float4*>(&red[w][col]);
        s.x += x.x; s.y += x.y; s.z += x.z; s.w += x.w;
      }
      const float4 vv = *reinterpret_cast<const float4*>(&vs[col]);
      r.x = beta * (vv.x - s.x); r.y = beta * (vv.y - s.y); r.z = beta * (vv.z - s.z); r.w = beta * (vv.w - s.w);
    }
    __syncthreads();   // every warp has read the partial sums before they are overwritten below
    float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int i = 0; i < RW; ++i) {
      const float kk = ks[r0 + i] * kn, qq = qs[r0 + i] * qn;
      st[i].x += kk * r.x; st[i].y += kk * r.y; st[i].z += kk * r.z; st[i].w += kk * r.w;
      o.x += st[i].x * qq; o.y += st[i].y * qq; o.z += st[i].z * qq; o.w += st[i].w * qq;
    }
    *reinterpret_cast<float4*>(&red[warp][col]) = o;
    __syncthreads();
    if (tid < DV) {
      float s = 0.f;
#pragma unroll
      for (int w = 0; w < 8; ++w) s += red[w][tid];
      st_elem(a.o, (row * a.HV + hv) * DV + tid, a.qkv_dtype, s);
    }
  }

  if (ht != nullptr) {
#pragma unroll
    for (int i = 0; i < RW; ++i) *reinterpret_cast<float4*>(ht + (int64_t)(r0 + i) * DV + col) = st[i];
  }
}

// Single-token decode at large batch as a stream: the kernels above load a state, compute and store it, so the
// memory pipe of an SM idles while its CTAs compute.  Here one persistent CTA per SM walks its (sequence, head) items
// through a three-stage ring in shared memory: a producer warp brings each 64 KiB state (one contiguous bulk copy), the
// token's q, k, v rows and the activated gate scalars two items ahead and writes finished states back (one bulk copy);
// eight consumer warps only compute, shared memory to shared memory.  Every wait is bounded.
__device__ int g_decode_timeout = 0;

template <int DK>
struct DecodeSmem {
  static constexpr int NS = 3;
  static constexpr size_t state_bytes = (size_t)DK * 128 * 4;
  static constexpr size_t o_q = state_bytes, o_k = o_q + 512, o_v = o_k + 512, o_sc = o_v + 512;
  static constexpr size_t stage = o_sc + 128;
  static constexpr size_t o_red = NS * stage;
  static constexpr size_t o_bar = o_red + 8 * 128 * 4;
  static constexpr size_t bytes = o_bar + 128;
};

template <int DK>
__global__ void __launch_bounds__(288, 1) decode_stream_kernel(const b200gdn_recurrent_args a, const int n_items) {
  using S = DecodeSmem<DK>;
  constexpr int NS = S::NS, DV = 128, RW = DK / 8;
  extern __shared__ __align__(128) unsigned char dsm[];
  float (*red)[DV] = reinterpret_cast<float (*)[DV]>(dsm + S::o_red);
  uint64_t* full = reinterpret_cast<uint64_t*>(dsm + S::o_bar);
  uint64_t* done = full + NS;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int esz = a.qkv_dtype == 2 ? 4 : 2;
  const int n_local = (n_items - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;
  const int G = a.HV / a.H;

  if (tid == 0) {
    for (int s = 0; s < NS; ++s) {
      tc5::mbar_init(&full[s], 1);
      tc5::mbar_init(&done[s], 256);
    }
    tc5::fence_mbar_init();
  }
  __syncthreads();

  if (warp == 8) {
    // ---- producer: write-back of the item that used the stage last, then the load of the item NS further on
    if (lane == 0) {
      bool failed = false;
      for (int jj = 0; jj < n_local + NS && !failed; ++jj) {
        const int s = jj % NS;
        unsigned char* stg = dsm + (size_t)s * S::stage;
        if (jj >= NS) {
          const int item = (int)blockIdx.x + (jj - NS) * (int)gridDim.x;
          if (!tc5::mbar_wait(&done[s], ((jj - NS) / NS) & 1)) { failed = true; break; }
          bool writeback;
          const int64_t slot = state_slot(a, item / a.HV, &writeback);
          if (writeback) {
            float* ht = a.ht + (slot * a.HV + item % a.HV) * DK * DV;
            asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;\n" ::"l"(ht), "r"(tc5::smem_addr(stg)),
                         "r"((uint32_t)S::state_bytes)
                         : "memory");
            tma::store_commit();
            tma::store_wait_read<0>();   // the stage may be refilled once the copy has read it
          }
        }
        if (jj < n_local) {
          const int item = (int)blockIdx.x + jj * (int)gridDim.x;
          const int n = item / a.HV, hv = item % a.HV, hq = hv / G;
          const int64_t row = n;   // one token per sequence
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
          float* sc = reinterpret_cast<float*>(stg + S::o_sc);
          sc[0] = expf(gg);
          sc[1] = bb;
          const uint32_t qk_bytes = (uint32_t)(DK * esz), v_bytes = (uint32_t)(DV * esz);
          tc5::mbar_expect_tx(&full[s], (uint32_t)S::state_bytes + 2 * qk_bytes + v_bytes);
          bool writeback_unused;
          const int64_t slot = state_slot(a, n, &writeback_unused);
          tma::load_1d(stg, a.h0 + (slot * a.HV + hv) * DK * DV, (uint32_t)S::state_bytes, &full[s]);
          tma::load_1d(stg + S::o_q, static_cast<const char*>(a.q) + (row * a.H + hq) * DK * esz, qk_bytes, &full[s]);
          tma::load_1d(stg + S::o_k, static_cast<const char*>(a.k) + (row * a.H + hq) * DK * esz, qk_bytes, &full[s]);
          tma::load_1d(stg + S::o_v, static_cast<const char*>(a.v) + (row * a.HV + hv) * DV * esz, v_bytes, &full[s]);
        }
      }
      tma::store_wait_all<0>();
      if (failed) atomicExch(&g_decode_timeout, 1);
    }
    return;
  }

  // ---- consumers (8 warps): warp w keeps rows [w RW, (w+1) RW), lane l the columns 4 l .. 4 l + 3
  const int col = 4 * lane, r0 = warp * RW;
  auto sync_consumers = [] { asm volatile("bar.sync 1, 256;\n" ::: "memory"); };
  for (int j = 0; j < n_local; ++j) {
    const int s = j % NS;
    unsigned char* stg = dsm + (size_t)s * S::stage;
    float* St = reinterpret_cast<float*>(stg);
    const int item = (int)blockIdx.x + j * (int)gridDim.x;
    const int hv = item % a.HV;
    {
      // the consumers agree on the outcome of the bounded wait (a barrier-wide OR), so that they leave together;
      // the producer then gives up on its own bounded wait
      const uint32_t bad = tc5::mbar_wait(&full[s], (j / NS) & 1) ? 0u : 1u;
      uint32_t any_bad;
      asm volatile(
          "{\n.reg .pred p, q;\nsetp.ne.b32 q, %1, 0;\nbar.red.or.pred p, 1, 256, q;\nselp.u32 %0, 1, 0, p;\n}\n"
          : "=r"(any_bad)
          : "r"(bad)
          : "memory");
      if (any_bad) {
        if (tid == 0) atomicExch(&g_decode_timeout, 1);
        return;
      }
    }
    const float* sc = reinterpret_cast<const float*>(stg + S::o_sc);
    const float decay = sc[0], beta = sc[1];
    float qn = a.scale, kn = 1.f;
    if (a.flags & B200GDN_REC_L2NORM) {
      float sq = 0.f, sk = 0.f;
      for (int i = lane; i < DK; i += 32) {
        const float x = ld_elem(stg + S::o_q, i, a.qkv_dtype), y = ld_elem(stg + S::o_k, i, a.qkv_dtype);
        sq += x * x;
        sk += y * y;
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        sq += __shfl_xor_sync(0xffffffffu, sq, o);
        sk += __shfl_xor_sync(0xffffffffu, sk, o);
      }
      qn = a.scale * rsqrtf(sq + 1e-6f);
      kn = rsqrtf(sk + 1e-6f);
    }
    float4 st[RW];
    float kr[RW];
    float4 d = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int i = 0; i < RW; ++i) {
      st[i] = *reinterpret_cast<const float4*>(St + (r0 + i) * DV + col);
      kr[i] = ld_elem(stg + S::o_k, r0 + i, a.qkv_dtype) * kn;
      st[i].x *= decay; st[i].y *= decay; st[i].z *= decay; st[i].w *= decay;
      d.x += st[i].x * kr[i]; d.y += st[i].y * kr[i]; d.z += st[i].z * kr[i]; d.w += st[i].w * kr[i];
    }
    *reinterpret_cast<float4*>(&red[warp][col]) = d;
    sync_consumers();
    float4 r;
    {
      float4 sum = *reinterpret_cast<const float4*>(&red[0][col]);
#pragma unroll
      for (int w = 1; w < 8; ++w) {
        const float4 x = *reinterpret_cast<const float4*>(&red[w][col]);
        sum.x += x.x; sum.y += x.y; sum.z += x.z; sum.w += x.w;
      }
      const float v0 = ld_elem(stg + S::o_v, col, a.qkv_dtype), v1 = ld_elem(stg + S::o_v, col + 1, a.qkv_dtype);
      const float v2 = ld_elem(stg + S::o_v, col + 2, a.qkv_dtype), v3 = ld_elem(stg + S::o_v, col + 3, a.qkv_dtype);
      r.x = beta * (v0 - sum.x); r.y = beta * (v1 - sum.y); r.z = beta * (v2 - sum.z); r.w = beta * (v3 - sum.w);
    }
    sync_consumers();   // the partial sums have been read by everybody before they are overwritten
    float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int i = 0; i < RW; ++i) {
      const float qq = ld_elem(stg + S::o_q, r0 + i, a.qkv_dtype) * qn;
      st[i].x += kr[i] * r.x; st[i].y += kr[i] * r.y; st[i].z += kr[i] * r.z; st[i].w += kr[i] * r.w;
      o.x += st[i].x * qq; o.y += st[i].y * qq; o.z += st[i].z * qq; o.w += st[i].w * qq;
      *reinterpret_cast<float4*>(St + (r0 + i) * DV + col) = st[i];
    }
    *reinterpret_cast<float4*>(&red[warp][col]) = o;
    tc5::fence_async_smem();       // the new state is read by the producer's bulk copy
    sync_consumers();
    if (tid < DV) {
      float sum = 0.f;
#pragma unroll
      for (int w = 0; w < 8; ++w) sum += red[w][tid];
      st_elem(a.o, ((int64_t)(item / a.HV) * a.HV + hv) * DV + tid, a.qkv_dtype, sum);
    }
    tc5::mbar_arrive(&done[s]);
    sync_consumers();   // red is free again for the next item
  }
}

template <int DK>
int launch(const b200gdn_recurrent_args& a, cudaStream_t st) {
  if constexpr (DK == 64 || DK == 128) {
    // one token per sequence at large batch: the streaming kernel (state and token rows by bulk copies, ring of three)
    if (!(a.flags & B200GDN_REC_STATE_V_FIRST) && a.V == 128 && a.T == 1 && a.cu_seqlens == nullptr && a.h0 != nullptr &&
        a.ht != nullptr && (int64_t)a.n_seq * a.HV >= 256 && (reinterpret_cast<uintptr_t>(a.q) & 15) == 0 &&
        (reinterpret_cast<uintptr_t>(a.k) & 15) == 0 && (reinterpret_cast<uintptr_t>(a.v) & 15) == 0 &&
        (reinterpret_cast<uintptr_t>(a.h0) & 15) == 0 && (reinterpret_cast<uintptr_t>(a.ht) & 15) == 0) {
      using S = DecodeSmem<DK>;
      if (int e = ensure_smem(decode_stream_kernel<DK>, S::bytes)) return e;
      int dev = 0, sms = 148;
      cudaGetDevice(&dev);
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
      const int n_items = a.n_seq * a.HV;
      decode_stream_kernel<DK><<<n_items < sms ? n_items : sms, 288, S::bytes, st>>>(a, n_items);
      return check_launch("decode_stream");
    }
    // whole-state CTAs (contiguous state traffic) once there are enough (sequence, head) pairs to fill the GPU;
    // smaller problems keep the four-times finer slicing of the kernel above
    if (!(a.flags & B200GDN_REC_STATE_V_FIRST) && a.V == 128 && (int64_t)a.n_seq * a.HV >= 256) {
      recurrent_rows_kernel<DK><<<dim3(a.HV, a.n_seq), 256, 0, st>>>(a);
      return check_launch("recurrent_rows");
    }
  }
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

// Reads and clears the flag a bounded device wait raises when it expires (synchronises with the device).
int decode_timeout_flag() {
  int v = 0, zero = 0;
  cudaMemcpyFromSymbol(&v, g_decode_timeout, sizeof(int));
  if (v) cudaMemcpyToSymbol(g_decode_timeout, &zero, sizeof(int));
  return v;
}

}  // namespace gdn
