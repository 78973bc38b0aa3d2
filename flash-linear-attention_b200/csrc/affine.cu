// out = M x + b (or M^T x + b) per head, fp32: folds a received state prefix through a shard's K x K
// transition matrix for context parallelism (merge step of fla/ops/cp/chunk_delta_h.py:332-460).
// Tiny (2 K^2 V flop per head), so a plain shared-memory tiled fp32 kernel: exact fp32 keeps the
// chained prefix as accurate as the reference's fp32 merge.
#include "gdn_common.cuh"

namespace gdn {
namespace {

constexpr int TM = 64, TN = 64, TK = 16;

__global__ void __launch_bounds__(256) affine_kernel(const b200gdn_affine_args a) {
  __shared__ float Ms[TK][TM + 1];
  __shared__ float Xs[TK][TN + 1];
  const int hv = blockIdx.z, i0 = blockIdx.y * TM, j0 = blockIdx.x * TN;
  const int K = a.K, V = a.V;
  const float* M = a.M + (int64_t)hv * K * K;
  const float* x = a.x + (int64_t)hv * K * V;
  const int tid = threadIdx.x, ty = tid / 16, tx = tid % 16;
  float acc[4][4] = {};
  for (int m0 = 0; m0 < K; m0 += TK) {
    for (int idx = tid; idx < TK * TM; idx += 256) {
      int mm = idx / TM, ii = idx % TM;
      int gi = i0 + ii, gm = m0 + mm;
      float val = 0.f;
      if (gi < K && gm < K) val = a.transpose_m ? M[(int64_t)gm * K + gi] : M[(int64_t)gi * K + gm];
      Ms[mm][ii] = val;
    }
    for (int idx = tid; idx < TK * TN; idx += 256) {
      int mm = idx / TN, jj = idx % TN;
      int gm = m0 + mm, gj = j0 + jj;
      Xs[mm][jj] = (gm < K && gj < V) ? x[(int64_t)gm * V + gj] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int mm = 0; mm < TK; ++mm) {
      float am[4], bx[4];
#pragma unroll
      for (int r = 0; r < 4; ++r) am[r] = Ms[mm][ty * 4 + r];
#pragma unroll
      for (int c = 0; c < 4; ++c) bx[c] = Xs[mm][tx * 4 + c];
#pragma unroll
      for (int r = 0; r < 4; ++r)
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[r][c] += am[r] * bx[c];
    }
    __syncthreads();
  }
#pragma unroll
  for (int r = 0; r < 4; ++r)
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      int gi = i0 + ty * 4 + r, gj = j0 + tx * 4 + c;
      if (gi < K && gj < V) {
        int64_t o = (int64_t)hv * K * V + (int64_t)gi * V + gj;
        a.out[o] = acc[r][c] + (a.b ? a.b[o] : 0.f);
      }
    }
}

// The whole prefix fold of a rank in one launch: x = b_first; then x = M_j x + b_j for the following `count - 1`
// ranks j = first + step, first + 2 step, ... of the gathered pairs [world][HV][K][K + V] (M in columns [0, K), the
// state part in [K, K + V)), written to out [HV][K][V].  A CTA owns one head and CS value columns (the chain of a
// column slice is independent of the other columns) and keeps its x slice in shared memory; 2 threads per row.
constexpr int CS = 32;

__global__ void cp_fold_kernel(const b200gdn_fold_args a) {
  extern __shared__ float xs[];   // [2][K][CS]
  const int K = a.K, V = a.V, hv = blockIdx.y, c0 = blockIdx.x * CS;
  const int64_t stride = K + V;
  const int tid = threadIdx.x, r = tid >> 1, ch = (tid & 1) * (CS / 2);
  auto pair = [&](int j) { return a.gathered + ((int64_t)j * a.HV + hv) * K * stride; };
  const float* P = pair(a.first);
  float acc[CS / 2];
#pragma unroll
  for (int c = 0; c < CS / 2; ++c) {
    acc[c] = P[r * stride + K + c0 + ch + c];
    xs[r * CS + ch + c] = acc[c];
  }
  __syncthreads();
  int cur = 0;
  for (int i = 1; i < a.count; ++i) {
    P = pair(a.first + i * a.step);
    const float* x = xs + cur * K * CS;
#pragma unroll
    for (int c = 0; c < CS / 2; ++c) acc[c] = P[r * stride + K + c0 + ch + c];
    for (int m = 0; m < K; m += 4) {
      const float4 mv = *reinterpret_cast<const float4*>(&P[r * stride + m]);
      const float mm[4] = {mv.x, mv.y, mv.z, mv.w};
#pragma unroll
      for (int e = 0; e < 4; ++e)
#pragma unroll
        for (int c = 0; c < CS / 2; ++c) acc[c] += mm[e] * x[(m + e) * CS + ch + c];
    }
    float* y = xs + (cur ^ 1) * K * CS;
#pragma unroll
    for (int c = 0; c < CS / 2; ++c) y[r * CS + ch + c] = acc[c];
    __syncthreads();
    cur ^= 1;
  }
#pragma unroll
  for (int c = 0; c < CS / 2; ++c) a.out[((int64_t)hv * K + r) * V + c0 + ch + c] = acc[c];
}

// Chains of affine maps inside one GPU (a long sequence cut into pieces that are scanned concurrently): for every
// chain c of the table, x = x0[c] (zeros, or the identity when x0 == NULL and identity != 0); out[first_out] = x; then
// for t = 0 .. count-2:  x = M[j_t] x + h[j_t],  out[o_t] = x, with
//   forward:  j_t = first_pre + t,              o_t = first_out + t + 1
//   reverse:  j_t = first_pre + count - 2 - t,  o_t = first_out + count - 2 - t   (out[first_out + count - 1] = x0 first)
// and, when `last` is given, last[c] = the chain's final x.  Same thread layout as the fold above.
__global__ void cp_prefix_kernel(const b200gdn_prefix_args a) {
  extern __shared__ float xs[];   // [2][K][CS]
  const int K = a.K, V = a.V, hv = blockIdx.y, c0 = blockIdx.x * CS, chain = blockIdx.z;
  const int tid = threadIdx.x, r = tid >> 1, ch = (tid & 1) * (CS / 2);
  const int first_out = a.table[3 * chain], count = a.table[3 * chain + 1], first_pre = a.table[3 * chain + 2];
  float acc[CS / 2];
#pragma unroll
  for (int c = 0; c < CS / 2; ++c) {
    const int col = c0 + ch + c;
    acc[c] = a.x0 ? a.x0[(((int64_t)chain * a.HV + hv) * K + r) * V + col] : ((a.identity && r == col) ? 1.f : 0.f);
    xs[r * CS + ch + c] = acc[c];
  }
  auto emit = [&](int piece) {
    if (a.out == nullptr) return;
#pragma unroll
    for (int c = 0; c < CS / 2; ++c) a.out[(((int64_t)piece * a.HV + hv) * K + r) * V + c0 + ch + c] = acc[c];
  };
  emit(a.reverse ? first_out + count - 1 : first_out);
  __syncthreads();
  int cur = 0;
  for (int t = 0; t + 1 < count; ++t) {
    const int j = a.reverse ? first_pre + count - 2 - t : first_pre + t;
    const float* M = a.M + ((int64_t)j * a.HV + hv) * K * K;
    const float* x = xs + cur * K * CS;
#pragma unroll
    for (int c = 0; c < CS / 2; ++c) acc[c] = a.h ? a.h[(((int64_t)j * a.HV + hv) * K + r) * V + c0 + ch + c] : 0.f;
    for (int m = 0; m < K; m += 4) {
      const float4 mv = *reinterpret_cast<const float4*>(&M[r * K + m]);
      const float mm[4] = {mv.x, mv.y, mv.z, mv.w};
#pragma unroll
      for (int e = 0; e < 4; ++e)
#pragma unroll
        for (int c = 0; c < CS / 2; ++c) acc[c] += mm[e] * x[(m + e) * CS + ch + c];
    }
    float* y = xs + (cur ^ 1) * K * CS;
#pragma unroll
    for (int c = 0; c < CS / 2; ++c) y[r * CS + ch + c] = acc[c];
    emit(a.reverse ? first_out + count - 2 - t : first_out + t + 1);
    __syncthreads();
    cur ^= 1;
  }
  if (a.last != nullptr) {
#pragma unroll
    for (int c = 0; c < CS / 2; ++c) a.last[(((int64_t)chain * a.HV + hv) * K + r) * V + c0 + ch + c] = acc[c];
  }
}

}  // namespace

int launch_cp_prefix(const b200gdn_prefix_args& a, cudaStream_t st) {
  const size_t smem = (size_t)2 * a.K * CS * sizeof(float);
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(cp_prefix_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return set_error(B200GDN_ERR_CUDA, "cp_prefix: %s", cudaGetErrorString(e));
  }
  dim3 grid(a.V / CS, a.HV, a.n_chains);
  cp_prefix_kernel<<<grid, 2 * a.K, smem, st>>>(a);
  return check_launch("cp_prefix");
}

int launch_cp_fold(const b200gdn_fold_args& a, cudaStream_t st) {
  const size_t smem = (size_t)2 * a.K * CS * sizeof(float);
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(cp_fold_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return set_error(B200GDN_ERR_CUDA, "cp_fold: %s", cudaGetErrorString(e));
  }
  dim3 grid(a.V / CS, a.HV);
  cp_fold_kernel<<<grid, 2 * a.K, smem, st>>>(a);
  return check_launch("cp_fold");
}

int launch_affine(const b200gdn_affine_args& a, cudaStream_t st) {
  dim3 grid((a.V + TN - 1) / TN, (a.K + TM - 1) / TM, a.HV);
  affine_kernel<<<grid, 256, 0, st>>>(a);
  return check_launch("affine_apply");
}

}  // namespace gdn
