// C ABI of the library (declared in include/b200gdn.h): argument checks, stage sequencing, error text.
#include <cstdarg>
#include <cstdio>

#include "gdn_common.cuh"
#include "tc5.cuh"

namespace gdn {

static thread_local char g_err[512] = "";
static thread_local int g_launches = 0;

int set_error(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

void reset_launch_count() { g_launches = 0; }

int check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return set_error(B200GDN_ERR_CUDA, "%s launch: %s", what, cudaGetErrorString(e));
  ++g_launches;
  return 0;
}

static int check_chunk_args(const b200gdn_chunk_args* a, const char* who) {
  if (a == nullptr) return set_error(B200GDN_ERR_BAD_ARGUMENT, "%s: args is NULL", who);
  if (a->struct_bytes != (int32_t)sizeof(b200gdn_chunk_args))
    return set_error(B200GDN_ERR_BAD_ARGUMENT, "%s: struct_bytes %d != %zu (ABI mismatch)", who, a->struct_bytes,
                     sizeof(b200gdn_chunk_args));
  if (a->rows <= 0 || a->H <= 0 || a->HV <= 0 || a->n_seq <= 0 || a->n_chunks <= 0)
    return set_error(B200GDN_ERR_BAD_ARGUMENT, "%s: empty problem (rows=%d H=%d HV=%d n_seq=%d n_chunks=%d)", who, a->rows,
                     a->H, a->HV, a->n_seq, a->n_chunks);
  if (a->HV % a->H != 0) return set_error(B200GDN_ERR_BAD_ARGUMENT, "%s: HV=%d not a multiple of H=%d", who, a->HV, a->H);
  if (a->chunk_meta == nullptr || a->seq_meta == nullptr)
    return set_error(B200GDN_ERR_BAD_ARGUMENT, "%s: chunk tables missing", who);
  if (a->HV > 65535 || a->n_seq > 65535)
    return set_error(B200GDN_ERR_UNSUPPORTED, "%s: HV and n_seq are grid y/z dimensions (<= 65535)", who);
  return 0;
}

#define REQUIRE(ptr, who)                                                                  \
  if ((ptr) == nullptr) return gdn::set_error(B200GDN_ERR_BAD_ARGUMENT, "%s: %s is NULL", who, #ptr)

}  // namespace gdn

namespace gdn {
__device__ int g_selftest_timeout = 0;
// One warp waits on an mbarrier that nothing will ever complete, with a short limit: the wait must give up, raise the
// flag and let the kernel end normally (what every wait of the real kernels does when a completion is lost).
__global__ void selftest_wait_expiry_kernel(uint32_t limit) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    tc5::mbar_init(&bar, 1);
    tc5::fence_mbar_init();
  }
  __syncthreads();
  const bool ok = tc5::mbar_wait(&bar, 0, limit);
  if (!ok && threadIdx.x == 0) atomicExch(&g_selftest_timeout, 1);
}
static int selftest_timeout_flag() {
  int v = 0, zero = 0;
  cudaMemcpyFromSymbol(&v, g_selftest_timeout, sizeof(int));
  if (v) cudaMemcpyToSymbol(g_selftest_timeout, &zero, sizeof(int));
  return v;
}
}  // namespace gdn

extern "C" {

int b200gdn_chunk_fwd(const b200gdn_chunk_args* a, void* stream) {
  using namespace gdn;
  g_launches = 0;
  if (int e = check_chunk_args(a, "chunk_fwd")) return e;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const uint32_t m = a->stage_mask ? a->stage_mask : (B200GDN_FWD_INTRA | B200GDN_FWD_SCAN | B200GDN_FWD_OUT);
  if (m & B200GDN_FWD_INTRA) {
    REQUIRE(a->k, "chunk_fwd"); REQUIRE(a->v, "chunk_fwd"); REQUIRE(a->g, "chunk_fwd"); REQUIRE(a->beta, "chunk_fwd");
    REQUIRE(a->gamma, "chunk_fwd"); REQUIRE(a->A, "chunk_fwd"); REQUIRE(a->w, "chunk_fwd"); REQUIRE(a->u, "chunk_fwd");
    if (int e = launch_intra_fwd(*a, st)) return e;
  }
  if ((m & B200GDN_FWD_SCAN) && (m & B200GDN_FWD_OUT)) {
    // the scan forms the output itself from the tiles it holds on chip: h and v_new are written for the backward
    // pass only (either may be NULL when no backward pass follows)
    REQUIRE(a->k, "chunk_fwd"); REQUIRE(a->w, "chunk_fwd"); REQUIRE(a->gamma, "chunk_fwd");
    REQUIRE(a->q, "chunk_fwd"); REQUIRE(a->o, "chunk_fwd");
    if (int e = launch_scan_out_fwd(*a, st)) return e;
    return 0;
  }
  if (m & B200GDN_FWD_SCAN) {
    REQUIRE(a->k, "chunk_fwd"); REQUIRE(a->w, "chunk_fwd"); REQUIRE(a->gamma, "chunk_fwd");
    if (int e = launch_scan_fwd(*a, st)) return e;
  }
  if (m & B200GDN_FWD_OUT) {
    REQUIRE(a->q, "chunk_fwd"); REQUIRE(a->k, "chunk_fwd"); REQUIRE(a->v_new, "chunk_fwd"); REQUIRE(a->h, "chunk_fwd");
    REQUIRE(a->gamma, "chunk_fwd"); REQUIRE(a->o, "chunk_fwd");
    if (int e = launch_out_fwd(*a, st)) return e;
  }
  return 0;
}

int b200gdn_chunk_bwd(const b200gdn_chunk_args* a, void* stream) {
  using namespace gdn;
  g_launches = 0;
  if (int e = check_chunk_args(a, "chunk_bwd")) return e;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const uint32_t m =
      a->stage_mask ? a->stage_mask : (B200GDN_BWD_DVLOCAL | B200GDN_BWD_SCAN | B200GDN_BWD_DQKWG | B200GDN_BWD_WY);
  if ((m & B200GDN_BWD_DVLOCAL) && (m & B200GDN_BWD_SCAN)) {
    // the reverse scan forms the chunk-local part of dv itself from the tiles it holds on chip; dv2 is an output only
    // (NULL: not stored, e.g. when only dh0 of a shard is wanted)
    REQUIRE(a->q, "chunk_bwd"); REQUIRE(a->k, "chunk_bwd"); REQUIRE(a->w, "chunk_bwd"); REQUIRE(a->gamma, "chunk_bwd");
    REQUIRE(a->d_o, "chunk_bwd");
    if (int e = launch_scan_dvl_bwd(*a, st)) return e;
  } else {
    if (m & B200GDN_BWD_DVLOCAL) {
      REQUIRE(a->q, "chunk_bwd"); REQUIRE(a->k, "chunk_bwd"); REQUIRE(a->gamma, "chunk_bwd"); REQUIRE(a->d_o, "chunk_bwd");
      REQUIRE(a->dv2, "chunk_bwd");
      if (int e = launch_dv_local(*a, st)) return e;
    }
    if (m & B200GDN_BWD_SCAN) {
      REQUIRE(a->k, "chunk_bwd"); REQUIRE(a->w, "chunk_bwd"); REQUIRE(a->gamma, "chunk_bwd");
      if (int e = launch_scan_bwd(*a, st)) return e;
    }
  }
  if (m & B200GDN_BWD_DQKWG) {
    REQUIRE(a->q, "chunk_bwd"); REQUIRE(a->k, "chunk_bwd"); REQUIRE(a->v_new, "chunk_bwd"); REQUIRE(a->gamma, "chunk_bwd");
    REQUIRE(a->h, "chunk_bwd"); REQUIRE(a->dh, "chunk_bwd"); REQUIRE(a->dv2, "chunk_bwd"); REQUIRE(a->d_o, "chunk_bwd");
    REQUIRE(a->dq, "chunk_bwd"); REQUIRE(a->dk, "chunk_bwd"); REQUIRE(a->dG, "chunk_bwd");
    if (int e = launch_bwd_dqk(*a, st)) return e;
  }
  if (m & B200GDN_BWD_WY) {
    REQUIRE(a->k, "chunk_bwd"); REQUIRE(a->v, "chunk_bwd"); REQUIRE(a->beta, "chunk_bwd"); REQUIRE(a->gamma, "chunk_bwd");
    REQUIRE(a->A, "chunk_bwd"); REQUIRE(a->h, "chunk_bwd"); REQUIRE(a->dv2, "chunk_bwd");
    REQUIRE(a->dG, "chunk_bwd"); REQUIRE(a->dk, "chunk_bwd"); REQUIRE(a->dv, "chunk_bwd"); REQUIRE(a->dg, "chunk_bwd");
    REQUIRE(a->dbeta, "chunk_bwd");
    if (int e = launch_bwd_wy(*a, st)) return e;
  }
  return 0;
}

int b200gdn_recurrent_fwd(const b200gdn_recurrent_args* a, void* stream) {
  using namespace gdn;
  g_launches = 0;
  if (a == nullptr) return set_error(B200GDN_ERR_BAD_ARGUMENT, "recurrent_fwd: args is NULL");
  if (a->struct_bytes != (int32_t)sizeof(b200gdn_recurrent_args))
    return set_error(B200GDN_ERR_BAD_ARGUMENT, "recurrent_fwd: struct_bytes %d != %zu (ABI mismatch)", a->struct_bytes,
                     sizeof(b200gdn_recurrent_args));
  if (a->B <= 0 || a->T <= 0 || a->H <= 0 || a->HV <= 0 || a->n_seq <= 0 || a->HV % a->H != 0)
    return set_error(B200GDN_ERR_BAD_ARGUMENT, "recurrent_fwd: bad sizes B=%d T=%d H=%d HV=%d n_seq=%d", a->B, a->T, a->H,
                     a->HV, a->n_seq);
  if (a->qkv_dtype < 0 || a->qkv_dtype > 2) return set_error(B200GDN_ERR_BAD_ARGUMENT, "recurrent_fwd: qkv_dtype %d", a->qkv_dtype);
  if (a->HV > 65535 || a->n_seq > 65535)
    return set_error(B200GDN_ERR_UNSUPPORTED, "recurrent_fwd: HV and n_seq are grid dimensions (<= 65535)");
  REQUIRE(a->q, "recurrent_fwd"); REQUIRE(a->k, "recurrent_fwd"); REQUIRE(a->v, "recurrent_fwd");
  REQUIRE(a->beta, "recurrent_fwd"); REQUIRE(a->o, "recurrent_fwd");
  return launch_recurrent(*a, static_cast<cudaStream_t>(stream));
}

int b200gdn_affine_apply(const b200gdn_affine_args* a, void* stream) {
  using namespace gdn;
  g_launches = 0;
  if (a == nullptr) return set_error(B200GDN_ERR_BAD_ARGUMENT, "affine_apply: args is NULL");
  if (a->struct_bytes != (int32_t)sizeof(b200gdn_affine_args))
    return set_error(B200GDN_ERR_BAD_ARGUMENT, "affine_apply: struct_bytes %d != %zu (ABI mismatch)", a->struct_bytes,
                     sizeof(b200gdn_affine_args));
  if (a->HV <= 0 || a->K <= 0 || a->V <= 0) return set_error(B200GDN_ERR_BAD_ARGUMENT, "affine_apply: bad sizes");
  REQUIRE(a->M, "affine_apply"); REQUIRE(a->x, "affine_apply"); REQUIRE(a->out, "affine_apply");
  return launch_affine(*a, static_cast<cudaStream_t>(stream));
}

int b200gdn_cp_fold(const b200gdn_fold_args* a, void* stream) {
  using namespace gdn;
  g_launches = 0;
  if (a == nullptr) return set_error(B200GDN_ERR_BAD_ARGUMENT, "cp_fold: args is NULL");
  if (a->struct_bytes != (int32_t)sizeof(b200gdn_fold_args))
    return set_error(B200GDN_ERR_BAD_ARGUMENT, "cp_fold: struct_bytes %d != %zu (ABI mismatch)", a->struct_bytes,
                     sizeof(b200gdn_fold_args));
  if (a->HV <= 0 || a->count < 1 || a->first < 0 || (a->step != 1 && a->step != -1) || a->first + (a->count - 1) * a->step < 0)
    return set_error(B200GDN_ERR_BAD_ARGUMENT, "cp_fold: bad sizes (HV=%d first=%d count=%d step=%d)", a->HV, a->first, a->count, a->step);
  if ((a->K != 64 && a->K != 128 && a->K != 256) || a->V <= 0 || a->V % 32 != 0)
    return set_error(B200GDN_ERR_UNSUPPORTED, "cp_fold: K=%d V=%d (K in {64,128,256}, V a multiple of 32)", a->K, a->V);
  REQUIRE(a->gathered, "cp_fold"); REQUIRE(a->out, "cp_fold");
  return launch_cp_fold(*a, static_cast<cudaStream_t>(stream));
}

int b200gdn_cp_prefix(const b200gdn_prefix_args* a, void* stream) {
  using namespace gdn;
  g_launches = 0;
  if (a == nullptr) return set_error(B200GDN_ERR_BAD_ARGUMENT, "cp_prefix: args is NULL");
  if (a->struct_bytes != (int32_t)sizeof(b200gdn_prefix_args))
    return set_error(B200GDN_ERR_BAD_ARGUMENT, "cp_prefix: struct_bytes %d != %zu (ABI mismatch)", a->struct_bytes,
                     sizeof(b200gdn_prefix_args));
  if (a->HV <= 0 || a->n_chains <= 0 || a->HV > 65535 || a->n_chains > 65535)
    return set_error(B200GDN_ERR_BAD_ARGUMENT, "cp_prefix: bad sizes (HV=%d n_chains=%d)", a->HV, a->n_chains);
  if ((a->K != 64 && a->K != 128 && a->K != 256) || a->V <= 0 || a->V % 32 != 0)
    return set_error(B200GDN_ERR_UNSUPPORTED, "cp_prefix: K=%d V=%d (K in {64,128,256}, V a multiple of 32)", a->K, a->V);
  REQUIRE(a->table, "cp_prefix"); REQUIRE(a->M, "cp_prefix");
  if (a->out == nullptr && a->last == nullptr) return set_error(B200GDN_ERR_BAD_ARGUMENT, "cp_prefix: no output given");
  return launch_cp_prefix(*a, static_cast<cudaStream_t>(stream));
}

int64_t b200gdn_saved_bytes(int32_t rows, int32_t H, int32_t HV, int32_t K, int32_t V, int32_t n_chunks) {
  (void)H;
  int64_t r = rows, hv = HV;
  return (int64_t)n_chunks * hv * 64 * 4  /* gamma */
         + r * hv * 64 * 2 * 2           /* A, qk */
         + r * hv * K * 2                /* w */
         + r * hv * V * 2 * 2            /* u, v_new */
         + (int64_t)n_chunks * hv * K * V * 2; /* h */
}

int64_t b200gdn_bwd_workspace_bytes(int32_t rows, int32_t H, int32_t HV, int32_t K, int32_t V, int32_t n_chunks) {
  int64_t r = rows, hv = HV;
  return (int64_t)n_chunks * hv * K * V * 2 /* dh */
         + r * hv * V * 2                    /* dv2 */
         + r * hv * 4                        /* dG */
         + (HV > H ? 2 * r * H * K * 4 : 0); /* dq_acc, dk_part: fp32 sums over a group of value heads */
}

static int check_prep_args(const b200gdn_prep_args* a, const char* who, bool bwd) {
  using namespace gdn;
  if (a == nullptr) return set_error(B200GDN_ERR_BAD_ARGUMENT, "%s: args is NULL", who);
  if (a->struct_bytes != (int32_t)sizeof(b200gdn_prep_args))
    return set_error(B200GDN_ERR_BAD_ARGUMENT, "%s: struct_bytes %d != %zu (ABI mismatch)", who, a->struct_bytes,
                     sizeof(b200gdn_prep_args));
  if (a->rows <= 0 || a->H <= 0 || a->HV <= 0) return set_error(B200GDN_ERR_BAD_ARGUMENT, "%s: bad sizes", who);
  if (a->qk_dtype < 0 || a->qk_dtype > 2 || a->gb_dtype < 0 || a->gb_dtype > 2)
    return set_error(B200GDN_ERR_BAD_ARGUMENT, "%s: dtype codes are 0 (bf16), 1 (fp16), 2 (fp32)", who);
  if (a->flags & B200GDN_PREP_L2NORM) {
    if (a->K != 64 && a->K != 128 && a->K != 256 && a->K != 512)
      return set_error(B200GDN_ERR_UNSUPPORTED, "%s: K=%d (64, 128, 256 and 512 are built)", who, a->K);
    REQUIRE(a->q, who); REQUIRE(a->k, who); REQUIRE(a->rstd_q, who); REQUIRE(a->rstd_k, who);
    if (!bwd) { REQUIRE(a->qn, who); REQUIRE(a->kn, who); }
    else { REQUIRE(a->dqn, who); REQUIRE(a->dkn, who); REQUIRE(a->dq, who); REQUIRE(a->dk, who); }
  }
  if (a->flags & B200GDN_PREP_GATE) {
    if (a->HV > 256) return set_error(B200GDN_ERR_UNSUPPORTED, "%s: HV=%d (at most 256 value heads)", who, a->HV);
    REQUIRE(a->g, who); REQUIRE(a->A_log, who);
    if (!bwd) { REQUIRE(a->g_out, who); }
    else { REQUIRE(a->dg, who); REQUIRE(a->dg_raw, who); REQUIRE(a->dA_log, who); REQUIRE(a->partials, who); }
  }
  if (a->flags & B200GDN_PREP_BETA_SIGMOID) {
    if (a->HV > 256) return set_error(B200GDN_ERR_UNSUPPORTED, "%s: HV=%d (at most 256 value heads)", who, a->HV);
    REQUIRE(a->beta, who);
    if (!bwd) { REQUIRE(a->beta_out, who); }
    else { REQUIRE(a->dbeta, who); REQUIRE(a->dbeta_raw, who); }
  }
  return 0;
}

int b200gdn_prep_fwd(const b200gdn_prep_args* a, void* stream) {
  gdn::g_launches = 0;
  if (int e = check_prep_args(a, "prep_fwd", false)) return e;
  return gdn::launch_prep(*a, static_cast<cudaStream_t>(stream), false);
}

int b200gdn_prep_bwd(const b200gdn_prep_args* a, void* stream) {
  gdn::g_launches = 0;
  if (int e = check_prep_args(a, "prep_bwd", true)) return e;
  return gdn::launch_prep(*a, static_cast<cudaStream_t>(stream), true);
}

static int check_conv_args(const b200gdn_conv_args* a, const char* who, bool bwd) {
  using namespace gdn;
  if (a == nullptr) return set_error(B200GDN_ERR_BAD_ARGUMENT, "%s: args is NULL", who);
  if (a->struct_bytes != (int32_t)sizeof(b200gdn_conv_args))
    return set_error(B200GDN_ERR_BAD_ARGUMENT, "%s: struct_bytes %d != %zu (ABI mismatch)", who, a->struct_bytes,
                     sizeof(b200gdn_conv_args));
  if (a->rows <= 0 || a->D <= 0 || a->n_seq <= 0 || a->n_tiles <= 0)
    return set_error(B200GDN_ERR_BAD_ARGUMENT, "%s: empty problem (rows=%d D=%d n_seq=%d n_tiles=%d)", who, a->rows, a->D, a->n_seq, a->n_tiles);
  if (a->D % 8 != 0) return set_error(B200GDN_ERR_UNSUPPORTED, "%s: D=%d is not a multiple of 8", who, a->D);
  if (a->W < 2 || a->W > 4) return set_error(B200GDN_ERR_UNSUPPORTED, "%s: kernel size %d (2, 3 and 4 are built)", who, a->W);
  if (a->dtype < 0 || a->dtype > 2) return set_error(B200GDN_ERR_BAD_ARGUMENT, "%s: dtype code %d", who, a->dtype);
  REQUIRE(a->tile_meta, who); REQUIRE(a->seq_meta, who); REQUIRE(a->x, who); REQUIRE(a->weight, who);
  if (!bwd) { REQUIRE(a->y, who); }
  else {
    REQUIRE(a->dy, who); REQUIRE(a->dx, who);
    if (a->dweight != nullptr) REQUIRE(a->partials, who);
  }
  return 0;
}

int b200gdn_conv_fwd(const b200gdn_conv_args* a, void* stream) {
  gdn::g_launches = 0;
  if (int e = check_conv_args(a, "conv_fwd", false)) return e;
  return gdn::launch_conv(*a, static_cast<cudaStream_t>(stream), false);
}

int b200gdn_conv_bwd(const b200gdn_conv_args* a, void* stream) {
  gdn::g_launches = 0;
  if (int e = check_conv_args(a, "conv_bwd", true)) return e;
  return gdn::launch_conv(*a, static_cast<cudaStream_t>(stream), true);
}

static int check_norm_gate_args(const b200gdn_norm_gate_args* a, const char* who, bool bwd) {
  using namespace gdn;
  if (a == nullptr) return set_error(B200GDN_ERR_BAD_ARGUMENT, "%s: args is NULL", who);
  if (a->struct_bytes != (int32_t)sizeof(b200gdn_norm_gate_args))
    return set_error(B200GDN_ERR_BAD_ARGUMENT, "%s: struct_bytes %d != %zu (ABI mismatch)", who, a->struct_bytes,
                     sizeof(b200gdn_norm_gate_args));
  if (a->rows <= 0) return set_error(B200GDN_ERR_BAD_ARGUMENT, "%s: empty problem", who);
  if (a->D != 64 && a->D != 128 && a->D != 256 && a->D != 512)
    return set_error(B200GDN_ERR_UNSUPPORTED, "%s: D=%d (64, 128, 256 and 512 are built)", who, a->D);
  if (a->dtype < 0 || a->dtype > 2) return set_error(B200GDN_ERR_BAD_ARGUMENT, "%s: dtype code %d", who, a->dtype);
  REQUIRE(a->x, who); REQUIRE(a->g, who); REQUIRE(a->rstd, who);
  if (!bwd) { REQUIRE(a->y, who); }
  else { REQUIRE(a->dy, who); REQUIRE(a->dx, who); REQUIRE(a->dg, who); REQUIRE(a->partials, who); }
  return 0;
}

int b200gdn_norm_gate_fwd(const b200gdn_norm_gate_args* a, void* stream) {
  gdn::g_launches = 0;
  if (int e = check_norm_gate_args(a, "norm_gate_fwd", false)) return e;
  return gdn::launch_norm_gate(*a, static_cast<cudaStream_t>(stream), false);
}

int b200gdn_norm_gate_bwd(const b200gdn_norm_gate_args* a, void* stream) {
  gdn::g_launches = 0;
  if (int e = check_norm_gate_args(a, "norm_gate_bwd", true)) return e;
  return gdn::launch_norm_gate(*a, static_cast<cudaStream_t>(stream), true);
}

int b200gdn_norm_gate_ctas(int64_t rows) { return gdn::norm_gate_grid(rows); }

int b200gdn_selftest_wait_expiry(void* stream) {
  gdn::g_launches = 0;
  gdn::selftest_wait_expiry_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(2000u);
  return gdn::check_launch("selftest_wait_expiry");
}

int b200gdn_device_status(void) {
  struct { const char* name; int (*flag)(); } k[] = {
      {"intra_fwd", gdn::intra_fwd_timeout_flag}, {"scan_fwd", gdn::scan_fwd_timeout_flag}, {"out_fwd", gdn::out_fwd_timeout_flag},
      {"dv_local", gdn::dv_local_timeout_flag},   {"scan_bwd", gdn::scan_bwd_timeout_flag}, {"bwd_dqk", gdn::bwd_dqk_timeout_flag},
      {"bwd_wy", gdn::bwd_wy_timeout_flag},       {"selftest", gdn::selftest_timeout_flag},
      {"decode_stream", gdn::decode_timeout_flag}};
  cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess) return gdn::set_error(B200GDN_ERR_CUDA, "device_status: %s", cudaGetErrorString(e));
  int rc = B200GDN_OK;
  for (auto& x : k)
    if (x.flag()) rc = gdn::set_error(B200GDN_ERR_TIMEOUT, "%s: a bounded device wait expired; its results are invalid", x.name);
  return rc;
}

int b200gdn_last_launch_count(void) { return gdn::g_launches; }
int b200gdn_abi_version(void) { return B200GDN_ABI_VERSION; }
const char* b200gdn_last_error(void) { return gdn::g_err; }

}  // extern "C"
