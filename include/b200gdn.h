/*
 * b200gdn — C ABI of the B200 (sm_100a) gated-delta-rule kernels.
 *
 * The reference (fla-org/flash-linear-attention 0.5.2) has no native ABI: its kernels are Triton
 * functions launched from Python.  Each entry point below replaces one Python-level orchestration
 * function of the reference; a backend plugin (fla/ops/backends/__init__.py:33-88, BaseBackend) or
 * any other host binds these symbols with ctypes / cffi / dlopen.
 *
 * Conventions
 *  - plain C: raw device pointers, 32-bit sizes, no torch types, no exceptions, no allocation
 *    (every buffer, including workspaces, is supplied by the caller);
 *  - every call only enqueues work on `stream` (a cudaStream_t passed as void*) of the CURRENT device
 *    and returns 0, or a negative b200gdn_status; b200gdn_last_error() gives the text;
 *  - token-major layout of the reference ([B,T,H,...], head_first is not supported) flattened to rows:
 *    q,k [rows,H,K]; v,o,do [rows,HV,V]; g,beta [rows,HV]; states [n_seq,HV,K,V] fp32;
 *    rows = B*T (dense) or the packed token count (cu_seqlens input, B == 1);
 *  - q/k/v/o/do and the saved tensors are bf16; gates, beta and states are fp32;
 *  - chunking (64 tokens, restarting at every sequence start) is described by two int32 tables that the
 *    host builds once per shape (fla/ops/utils/index.py:155-172 computes the same information):
 *      chunk_meta[n_chunks][4] = { sequence id, first row, valid rows (1..64), chunk index inside its sequence }
 *      seq_meta  [n_seq][2]    = { first chunk (global index), number of chunks }
 *  - the kernels move whole 64-row tiles: rows of a tile that lie past the end of a sequence are another
 *    sequence's rows or zero fill past the end of the tensor, and are selected away on chip.  Token rows that NO
 *    sequence covers (padding before the first or after the last sequence) are never written; when such rows
 *    exist the caller zero-fills the saved / workspace tensors once (w, u, v_new, dv2, A) and keeps the padding
 *    rows of q, k, v, do finite, because a tile load may bring them next to valid rows.
 */
#ifndef B200GDN_H_
#define B200GDN_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200GDN_ABI_VERSION 1
#define B200GDN_CHUNK 64

typedef enum b200gdn_status {
  B200GDN_OK = 0,
  B200GDN_ERR_BAD_ARGUMENT = -1,   /* null pointer, wrong struct size, zero size */
  B200GDN_ERR_UNSUPPORTED = -2,    /* head dimension / option not built */
  B200GDN_ERR_CUDA = -3,           /* a CUDA runtime call failed; see b200gdn_last_error() */
  B200GDN_ERR_TOO_LARGE = -4,      /* size exceeds a fixed capacity (static-scratch entry point) */
  B200GDN_ERR_TIMEOUT = -5         /* a bounded wait inside a kernel expired (b200gdn_device_status) */
} b200gdn_status;

/* stage masks: run only some kernels of a pass (unit tests and profiling); 0 means all */
#define B200GDN_FWD_INTRA 1u     /* gamma, A, w, u, qk     <- k, v, g, beta (, q) */
#define B200GDN_FWD_SCAN 2u      /* h, v_new, ht           <- k, w, u, gamma, h0 */
#define B200GDN_FWD_OUT 4u       /* o                      <- q, k, v_new, h, gamma */
#define B200GDN_BWD_DVLOCAL 1u   /* dv2 (local part)       <- q, k, gamma, do */
#define B200GDN_BWD_SCAN 2u      /* dh, dh0, dv2           <- q, k, w, gamma, do, dht */
#define B200GDN_BWD_DQKWG 4u     /* dq, dk (local part), dG <- q, k, v_new, gamma, h, dv2, do, dh */
#define B200GDN_BWD_WY 8u        /* dk, dv, dbeta, dg      <- k, v, beta, gamma, A, h, dv2, dk (local part), dG */

/* option bits shared by b200gdn_chunk_args.options and b200gdn_prep_args.flags (described with those structs) */
#define B200GDN_PREP_L2NORM 1u
#define B200GDN_PREP_GATE 2u
#define B200GDN_PREP_BETA_SIGMOID 4u
#define B200GDN_PREP_NEG_EIGVAL 8u
#define B200GDN_STATE_V_FIRST 16u /* chunk passes: h0, ht, dht and dh0 are stored [N,HV,V,K] (the reference's state_v_first) */
typedef struct b200gdn_chunk_args {
  int32_t struct_bytes;          /* = sizeof(b200gdn_chunk_args), checked */
  int32_t rows, H, HV, K, V;
  int32_t n_seq, n_chunks;
  float scale;
  uint32_t stage_mask;           /* 0 = all stages of the pass */
  const int32_t* chunk_meta;     /* device, [n_chunks][4] */
  const int32_t* seq_meta;       /* device, [n_seq][2] */
  /* inputs */
  const void* q;                 /* bf16 [rows,H,K] */
  const void* k;                 /* bf16 [rows,H,K] */
  const void* v;                 /* bf16 [rows,HV,V] */
  const float* g;                /* [rows,HV] log-space decay per token (forward only) */
  const float* beta;             /* [rows,HV] */
  const float* h0;               /* [n_seq,HV,K,V] or NULL */
  /* forward outputs */
  void* o;                       /* bf16 [rows,HV,V] */
  float* ht;                     /* [n_seq,HV,K,V] or NULL */
  /* written by the forward pass, read by the backward pass */
  float* gamma;                  /* [n_chunks,HV,64]  chunk-local cumsum(g) * log2(e); entries past a ragged
                                    chunk's length repeat the last valid value */
  void* A;                       /* bf16 [rows,HV,64]  rows of (I + L)^-1 */
  void* w;                       /* bf16 [rows,HV,K] */
  void* u;                       /* bf16 [rows,HV,V] */
  void* h;                       /* bf16 [n_chunks,HV,K,V]  state at each chunk start */
  void* v_new;                   /* bf16 [rows,HV,V] */
  /* backward inputs */
  const void* d_o;               /* bf16 [rows,HV,V] */
  const float* dht;              /* [n_seq,HV,K,V] or NULL */
  /* backward outputs */
  void* dq;                      /* bf16 [rows,H,K] */
  void* dk;                      /* bf16 [rows,H,K]; between B200GDN_BWD_DQKWG and B200GDN_BWD_WY it holds the
                                    chunk-local part of dk, to which the WY stage adds its terms in place */
  void* dv;                      /* bf16 [rows,HV,V] */
  float* dg;                     /* [rows,HV] */
  float* dbeta;                  /* [rows,HV] */
  float* dh0;                    /* [n_seq,HV,K,V] or NULL */
  /* backward workspace */
  void* dh;                      /* bf16 [n_chunks,HV,K,V] */
  void* dv2;                     /* bf16 [rows,HV,V] */
  void* dw;                      /* unused (dw = -dv2 h^T stays on chip); may be NULL */
  float* dk_part;                /* [rows,H,K], only read/written when HV > H (fp32 sum over a group's heads) */
  float* dG;                     /* [rows,HV] */
  float* dq_acc;                 /* [rows,H,K], only read/written when HV > H */
  /* The gate and beta options of the layer, fused (fla/ops/gated_delta_rule/gate.py:63-158, fla/ops/common/gate.py:18-50):
   * with B200GDN_PREP_GATE in `options`, g is the raw pre-activation and the kernels use
   * -exp(A_log) softplus(g + dt_bias); with B200GDN_PREP_BETA_SIGMOID (and B200GDN_PREP_NEG_EIGVAL), beta is raw and
   * the kernels use (1|2) sigmoid(beta).  dg / dbeta are then gradients w.r.t. the raw tensors, and the backward
   * also gives dA_log and ddt_bias.  options = 0: g and beta are used as they are. */
  uint32_t options;
  const float* A_log;            /* [HV] (GATE) */
  const float* dt_bias;          /* [HV] or NULL */
  float* gate_partials;          /* workspace fp32 [n_chunks,HV,2] (GATE, backward) */
  float* dA_log;                 /* out [HV] (GATE, backward) */
  float* ddt_bias;               /* out [HV] or NULL */
  /* Context parallelism (fla/ops/cp/chunk_delta_h.py:41-315, 478-744): with cp_M, the forward scan stage run alone
   * (B200GDN_FWD_SCAN) also gives, per scanned sequence, the K x K transition matrix M of S_end = M S_start + h_ext
   * (h_ext is what ht receives for a zero start state); with cp_dM the reverse scan gives the backward counterpart
   * next to dh0.  Both [n_seq,HV,K,K] fp32, NULL otherwise. */
  float* cp_M;
  float* cp_dM;
  /* written by the forward pass (intra stage, needs q), read by the fused scan stages of both passes:
   * bf16 [rows,HV,64], row i of a chunk holds <q_i,k_j> 2^(gamma_i - gamma_j) for j <= i, zero for j > i */
  void* qk;
  /* Backward only.  q / k as passed are the L2-normalised tensors b200gdn_prep_fwd produced
   * (fla/modules/l2norm.py:84-144); with their reciprocal norms given here (fp32 [rows,H]) the backward pass returns
   * dq / dk w.r.t. the un-normalised tensors, dx = (dy - y <dy,y>) rstd, applied where dq and dk are completed
   * (replaces l2norm_bwd, fla/modules/l2norm.py:200-251).  NULL: dq / dk are gradients w.r.t. q / k as passed. */
  const float* rstd_q;
  const float* rstd_k;
} b200gdn_chunk_args;

/* Replaces chunk_gated_delta_rule_fwd (fla/ops/gated_delta_rule/chunk.py:33-123):
 * chunk_local_cumsum + chunk_gated_delta_rule_fwd_intra + chunk_gated_delta_rule_fwd_h + chunk_fwd_o. */
int b200gdn_chunk_fwd(const b200gdn_chunk_args* args, void* stream);

/* No counterpart in the reference.  Same result as b200gdn_chunk_fwd (o and, when ht != NULL, the final state)
 * for callers that cannot allocate device memory (a server whose own pool already owns all of it, a plug-in
 * inside a foreign CUDA context, a C host that owns only inputs and outputs): the intermediate tensors live
 * in one array built into the library, B200GDN_STATIC_SCRATCH_BYTES bytes per GPU that loads the library, held
 * until exit.  The gamma/A/qk/w/u/h/v_new fields of `args` are ignored and nothing is saved for a backward pass.
 * Limit: align256(n_chunks*HV*256) + 2*align256(rows*HV*128) + align256(rows*HV*K*2) + align256(rows*HV*V*2)
 *        <=  B200GDN_STATIC_SCRATCH_BYTES
 * (e.g. 4096 tokens x 16 heads at K = V = 128); larger problems return B200GDN_ERR_TOO_LARGE and launch nothing.
 * Precondition (as for every chunk entry point): the sequences of the chunk tables cover all `rows` token rows.
 * Makes no allocating call.  The first call on each device looks up the array's address and should come before
 * any stream capture.  All calls on a device share the array (it keeps the previous call's contents; no stage
 * needs it cleared), so calls that can overlap on the GPU race: issue them in stream order. */
#define B200GDN_STATIC_SCRATCH_BYTES (64u << 20)
int b200gdn_chunk_fwd_static(const b200gdn_chunk_args* args, void* stream);

/* Replaces chunk_gated_delta_rule_bwd (fla/ops/gated_delta_rule/chunk.py:126-250):
 * chunk_bwd_dv_local + chunk_gated_delta_rule_bwd_dhu + chunk_bwd_dqkwg + prepare_wy_repr_bwd +
 * the reverse chunk_local_cumsum of dg.  Reads the tensors the forward pass saved. */
int b200gdn_chunk_bwd(const b200gdn_chunk_args* args, void* stream);

typedef struct b200gdn_recurrent_args {
  int32_t struct_bytes;
  int32_t B, T, H, HV, K, V;     /* dense: B sequences of T tokens; packed: B = 1, T = total tokens */
  int32_t n_seq;
  float scale;
  uint32_t flags;                /* B200GDN_REC_* */
  int32_t qkv_dtype;             /* 0 = bf16, 1 = fp16, 2 = fp32: element type of q, k, v and o */
  const int32_t* cu_seqlens;     /* device [n_seq+1] or NULL */
  const void* q;                 /* [B,T,H,K] */
  const void* k;                 /* [B,T,H,K] */
  const void* v;                 /* [B,T,HV,V] */
  const float* g;                /* [B,T,HV] or NULL */
  const float* beta;             /* [B,T,HV] */
  const float* A_log;            /* [HV] (gate in kernel) or NULL */
  const float* dt_bias;          /* [HV] or NULL */
  const float* h0;               /* [n_seq,HV,K,V] ([.,.,V,K] when V-first) or NULL */
  void* o;                       /* [B,T,HV,V] */
  float* ht;                     /* like h0, or NULL; may alias h0 for an in-place update */
  const int32_t* state_indices;  /* device [n_seq] or NULL.  No counterpart in the reference: with it, h0 and ht are
                                    pools of state slots [n_slots,HV,K,V] and sequence n uses slot state_indices[n]
                                    (the slots of one call must be distinct), as a serving engine's state cache
                                    addresses them; without it sequence n uses slot n */
  int32_t n_slots;               /* slots in the pool (with state_indices); an index outside [0, n_slots) marks a
                                    padding sequence: its state is neither taken from its slot nor written back and its
                                    output row is meaningless.  0 = unknown, indices are then trusted */
} b200gdn_recurrent_args;

#define B200GDN_REC_L2NORM 1u         /* q, k <- x * rsqrt(sum x^2 + 1e-6) */
#define B200GDN_REC_GATE 2u           /* g <- -exp(A_log) * softplus(g + dt_bias) */
#define B200GDN_REC_BETA_SIGMOID 4u   /* beta <- sigmoid(beta) */
#define B200GDN_REC_NEG_EIGVAL 8u     /* beta <- 2 * sigmoid(beta) (with BETA_SIGMOID) */
#define B200GDN_REC_STATE_V_FIRST 16u /* states stored [V,K] */

/* Replaces fused_recurrent_gated_delta_rule_fwd (fla/ops/gated_delta_rule/fused_recurrent.py:184-250). */
int b200gdn_recurrent_fwd(const b200gdn_recurrent_args* args, void* stream);

/* Context parallelism (fla/ops/cp/chunk_delta_h.py:747-936).  The transition of a whole shard is affine,
 * S_end = M S_start + h_ext; these produce M ([HV,K,K] fp32) for the rank's last (forward) or first
 * (backward) local sequence and fold a received prefix:  out = M x + b. */
typedef struct b200gdn_affine_args {
  int32_t struct_bytes;
  int32_t HV, K, V;
  int32_t transpose_m;           /* 0: out = M x + b ; 1: out = M^T x + b */
  const float* M;                /* [HV,K,K] */
  const float* x;                /* [HV,K,V] */
  const float* b;                /* [HV,K,V] or NULL */
  float* out;                    /* [HV,K,V] */
} b200gdn_affine_args;
int b200gdn_affine_apply(const b200gdn_affine_args* args, void* stream);

/* The prefix fold of one rank in a single launch (the chain of merges of fla/ops/cp/chunk_delta_h.py:332-460 over the
 * gathered pairs): x = b_first, then x = M_j x + b_j for j = first + step, ..., first + (count - 1) step, where rank
 * j's pair is gathered[j] = [HV, K, K + V] fp32 (M in columns [0, K), the state part b in [K, K + V)).
 * forward: first = rank - pre_num_ranks, step = +1;  backward (the pairs hold M^T): first = rank + post_num_ranks,
 * step = -1.  K in {64, 128, 256}, V a multiple of 32, count >= 1. */
typedef struct b200gdn_fold_args {
  int32_t struct_bytes;
  int32_t HV, K, V;
  int32_t first, count, step;
  const float* gathered;         /* [world, HV, K, K + V] */
  float* out;                    /* [HV, K, V] */
} b200gdn_fold_args;
int b200gdn_cp_fold(const b200gdn_fold_args* args, void* stream);

/* Prefix chains of affine maps inside one GPU: a long sequence is cut into pieces that are scanned concurrently (the
 * idea of fla/ops/common/intracard_cp.py:139-180 with the merge of fla/ops/cp/chunk_delta_h.py:254-315).  A pre-scan
 * gives piece j the pair (M[j], h[j]) with S_end = M[j] S_start + h[j]; this call turns them into the start state of
 * every piece.  For chain c (one sequence) with table[c] = {first_out, count, first_pre}:
 *   x = x0[c] (zeros when x0 == NULL; the identity when also `identity` != 0);  out[first_out] = x;
 *   for t = 0 .. count-2:  x = M[first_pre + t] x + h[first_pre + t];  out[first_out + t + 1] = x.
 * `reverse` walks the chain from its last piece to its first (the backward pass: out[first_out + count - 1] = x0,
 * pair first_pre + count - 2 - t, result into out[first_out + count - 2 - t]).  `last[c]`, when given, receives the
 * chain's final x (with h == NULL, identity and V == K: the product of the chain's matrices).
 * M [n_pre,HV,K,K], h [n_pre,HV,K,V], x0 / last [n_chains,HV,K,V], out [n_pieces,HV,K,V], all fp32;
 * K in {64,128,256}, V a multiple of 32. */
typedef struct b200gdn_prefix_args {
  int32_t struct_bytes;
  int32_t HV, K, V;
  int32_t n_chains, reverse, identity;
  const int32_t* table;          /* device [n_chains][3] */
  const float* M;
  const float* h;                /* or NULL (zeros) */
  const float* x0;               /* or NULL */
  float* out;                    /* or NULL */
  float* last;                   /* or NULL */
} b200gdn_prefix_args;
int b200gdn_cp_prefix(const b200gdn_prefix_args* args, void* stream);

/* The three options fla.layers.GatedDeltaNet turns on (fla/layers/gated_deltanet.py:309-325), as one pass before the
 * chunk kernels and one pass after their backward:
 *   L2NORM        y = x rsqrt(sum x^2 + 1e-6) over K for q and k, fp32 math; rstd saved
 *                 (l2norm_fwd_kernel / l2norm_bwd_kernel, fla/modules/l2norm.py:84-144)
 *   GATE          g = -exp(A_log) softplus(g_raw + dt_bias) per value head; backward also gives dA_log, ddt_bias
 *                 (gdn_gate_chunk_cumsum_scalar_kernel / gdn_gate_bwd_kernel, fla/ops/gated_delta_rule/gate.py:63-158;
 *                 the chunk cumulative sum itself stays inside b200gdn_chunk_fwd)
 *   BETA_SIGMOID  beta = s sigmoid(beta_raw), s = 2 with NEG_EIGVAL else 1
 *                 (fused_beta_sigmoid_fwd/bwd_kernel, fla/ops/common/gate.py:18-50)
 * Outputs the chunk entry points consume directly: q, k in bf16, g and beta in fp32.  An option that is off leaves
 * its outputs untouched (pass the raw tensor to the chunk call instead). */
#define B200GDN_PREP_PART_ROWS 128       /* rows of g reduced by one CTA of the backward pass */
typedef struct b200gdn_prep_args {
  int32_t struct_bytes;
  int32_t rows, H, HV, K;        /* K in {64, 128, 256, 512} */
  uint32_t flags;                /* B200GDN_PREP_* */
  int32_t qk_dtype;              /* 0 = bf16, 1 = fp16, 2 = fp32: element type of q, k, dq, dk */
  int32_t gb_dtype;              /* same code: element type of g, beta, dg_raw, dbeta_raw */
  const void* q;                 /* raw [rows,H,K] */
  const void* k;
  const void* g;                 /* raw [rows,HV] */
  const void* beta;              /* raw [rows,HV] */
  const float* A_log;            /* [HV] (GATE) */
  const float* dt_bias;          /* [HV] or NULL */
  void* qn;                      /* out bf16 [rows,H,K] (L2NORM) */
  void* kn;
  float* rstd_q;                 /* out [rows,H] (L2NORM) */
  float* rstd_k;
  float* g_out;                  /* out fp32 [rows,HV] (GATE) */
  float* beta_out;               /* out fp32 [rows,HV] (BETA_SIGMOID) */
  /* backward only */
  const void* dqn;               /* bf16 [rows,H,K]: gradients w.r.t. the normalised q, k */
  const void* dkn;
  const float* dg;               /* fp32 [rows,HV]: gradient w.r.t. the activated gate */
  const float* dbeta;            /* fp32 [rows,HV] */
  void* dq;                      /* out, qk_dtype [rows,H,K] */
  void* dk;
  void* dg_raw;                  /* out, gb_dtype [rows,HV] */
  void* dbeta_raw;               /* out, gb_dtype [rows,HV] */
  float* dA_log;                 /* out [HV] */
  float* ddt_bias;               /* out [HV] or NULL */
  float* partials;               /* workspace fp32 [ceil(rows / B200GDN_PREP_PART_ROWS), 2, HV] (GATE backward) */
} b200gdn_prep_args;
int b200gdn_prep_fwd(const b200gdn_prep_args* args, void* stream);
int b200gdn_prep_bwd(const b200gdn_prep_args* args, void* stream);

/* Short causal depthwise convolution (+ SiLU) on token-major activations, the step in front of the mixer
 * (fla/layers/gated_deltanet.py:247-300; causal_conv1d of fla/modules/conv/causal_conv1d.py:17-160 with the Triton
 * kernels of fla/modules/conv/triton/ops.py):  y[t,d] = act(bias[d] + sum_w weight[d,w] x[t-(W-1)+w, d]) (+ residual)
 * inside each sequence; x[-k] = initial_state[n,d,W-k] for k = 1..W-1 (zero without a cache); final_state[n,d,:] =
 * the last W inputs.  Tiles of up to 64 tokens of one sequence are described by the same two tables as the mixer's
 * chunks.  D a multiple of 8, W in {2,3,4}. */
#define B200GDN_CONV_SILU 1u
typedef struct b200gdn_conv_args {
  int32_t struct_bytes;
  int32_t rows, D, W;
  int32_t n_seq, n_tiles;
  uint32_t flags;                /* B200GDN_CONV_SILU */
  int32_t dtype;                 /* 0 = bf16, 1 = fp16, 2 = fp32: x, y, residual, states, dy, dx */
  const int32_t* tile_meta;      /* device [n_tiles][4], as chunk_meta */
  const int32_t* seq_meta;       /* device [n_seq][2], as seq_meta */
  const void* x;                 /* [rows, D] */
  const float* weight;           /* [D, W] */
  const float* bias;             /* [D] or NULL */
  const void* residual;          /* [rows, D] or NULL (forward) */
  const void* initial_state;     /* [n_seq, D, W] or NULL */
  void* y;                       /* [rows, D] (forward) */
  void* final_state;             /* [n_seq, D, W] or NULL (forward) */
  /* backward */
  const void* dy;                /* [rows, D] */
  void* dx;                      /* [rows, D] */
  float* dweight;                /* [D, W] or NULL */
  float* dbias;                  /* [D] or NULL */
  void* dinitial_state;          /* [n_seq, D, W] or NULL */
  float* partials;               /* workspace fp32 [2 n_tiles, D, W + 1]; required with dweight */
} b200gdn_conv_args;
int b200gdn_conv_fwd(const b200gdn_conv_args* args, void* stream);
int b200gdn_conv_bwd(const b200gdn_conv_args* args, void* stream);

/* Gated RMS norm over the head dimension, the step behind the mixer (fla/layers/gated_deltanet.py:355-357;
 * rms_norm_gated of fla/modules/fused_norm_gate.py:861-884 without residual):
 *   rstd = 1/sqrt(mean(x^2) + eps);  y = (x rstd weight + bias) act(g),  act = g sigmoid(g), or sigmoid(g) with
 * B200GDN_NORM_GATE_SIGMOID.  rows = tokens x heads, D in {64,128,256,512}.  The backward pass needs `partials`
 * of b200gdn_norm_gate_ctas(rows) x 2 x D floats. */
#define B200GDN_NORM_GATE_SIGMOID 1u
typedef struct b200gdn_norm_gate_args {
  int32_t struct_bytes;
  int32_t D;
  int64_t rows;
  uint32_t flags;
  int32_t dtype;                 /* 0 = bf16, 1 = fp16, 2 = fp32: x, g, y, dy, dx, dg */
  float eps;
  const void* x;                 /* [rows, D] */
  const void* g;                 /* [rows, D] */
  const float* weight;           /* [D] or NULL */
  const float* bias;             /* [D] or NULL */
  void* y;                       /* [rows, D] (forward) */
  float* rstd;                   /* [rows]: written by the forward pass, read by the backward pass */
  const void* dy;
  void* dx;
  void* dg;
  float* dweight;                /* [D] or NULL */
  float* dbias;                  /* [D] or NULL */
  float* partials;
} b200gdn_norm_gate_args;
int b200gdn_norm_gate_fwd(const b200gdn_norm_gate_args* args, void* stream);
int b200gdn_norm_gate_bwd(const b200gdn_norm_gate_args* args, void* stream);
int b200gdn_norm_gate_ctas(int64_t rows);

/* Bytes of forward-saved tensors and of backward workspace for a problem (what the caller allocates). */
int64_t b200gdn_saved_bytes(int32_t rows, int32_t H, int32_t HV, int32_t K, int32_t V, int32_t n_chunks);
int64_t b200gdn_bwd_workspace_bytes(int32_t rows, int32_t H, int32_t HV, int32_t K, int32_t V, int32_t n_chunks);

/* No counterpart in the reference (Triton kernels have no bounded waits).  Every wait inside the kernels of this
 * library (on an mbarrier that a TMA copy or a tensor-core commit completes) gives up after a fixed number of
 * polls, raises a flag in device memory and lets the CTA return, so that a lost completion cannot hang the GPU.
 * This call synchronises the device, reads and clears the flags of the current device and returns B200GDN_OK or
 * B200GDN_ERR_TIMEOUT (the results of the flagged kernel are then invalid; b200gdn_last_error() names it). */
int b200gdn_device_status(void);

/* No counterpart in the reference.  Launches one warp that waits, with a limit of 2000 polls, on an mbarrier nothing
 * completes: the wait gives up, raises the flag and the kernel ends normally.  The next b200gdn_device_status() then
 * returns B200GDN_ERR_TIMEOUT ("selftest") and the one after it B200GDN_OK: a host-side check that the expiry path of
 * the kernels' waits works and leaves the context usable, without faulting or hanging the GPU. */
int b200gdn_selftest_wait_expiry(void* stream);

/* Number of kernels the last call on this thread enqueued (bench bookkeeping). */
int b200gdn_last_launch_count(void);
int b200gdn_abi_version(void);
const char* b200gdn_last_error(void);

#ifdef __cplusplus
}
#endif
#endif /* B200GDN_H_ */
