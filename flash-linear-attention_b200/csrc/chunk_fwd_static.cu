// b200gdn_chunk_fwd_static: the forward pass for hosts that cannot allocate device memory.
//
// b200gdn_chunk_fwd needs intermediate tensors (gamma, A, qk, w, u, and for a backward pass h, v_new) that its caller has to
// allocate.  Some callers have no way to do that at call time: an inference server that handed all free
// device memory to its own pool at start-up and now finds cudaMalloc failing, a plug-in running inside
// another program's CUDA context with no agreed allocator, or a plain C host that only owns its input and
// output buffers.  For them this entry point keeps the intermediates in one fixed array that is part of
// the library image: B200GDN_STATIC_SCRATCH_BYTES bytes on every GPU on which the library's code is loaded,
// held until the process exits.  The caller passes inputs, chunk tables and outputs only.
//
// Nothing here calls cudaMalloc, cudaFree or any allocating library routine.
//
// The array is shared by every call on a device and keeps whatever the previous call left in it.  Nothing
// in the forward pass needs it to start at zero: each stage writes every element of a valid token row that a
// later stage uses.  (Full 64-row tile loads do touch rows beyond a ragged chunk's length: those are the next
// sequence's rows, or zero fill past the end of the tensor, and the kernels select them away.  This holds when
// the sequences of the chunk tables cover all `rows` token rows, which is a precondition of this entry point.)
// No clearing pass is run.  Two
// calls whose kernels can overlap on one GPU (different streams or different threads) race on the array
// and give wrong results: keep calls on a device in stream order.
//
// The first call on each device looks up the array's device address (cudaGetSymbolAddress); that first
// call should be made before any stream capture begins.
#include <mutex>

#include "gdn_common.cuh"

namespace {

// In host code this name is only a handle for the runtime's symbol table; it is NOT a device address.
// The address the kernels receive comes from cudaGetSymbolAddress below.
static __device__ __align__(256) unsigned char g_static_scratch[B200GDN_STATIC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
void* g_scratch_addr[kMaxDevices] = {};
void* g_scratch_ctx[kMaxDevices] = {};   // the CUDA context the cached address belongs to
std::mutex g_scratch_mutex;

// The current driver context (a second context on the same device has its own copy of the library image and
// therefore its own array); nullptr when the driver entry point cannot be resolved.
void* current_context() {
  typedef int (*CtxFn)(void**);
  static CtxFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuCtxGetCurrent", &p, cudaEnableDefault, &q) == cudaSuccess) fn = reinterpret_cast<CtxFn>(p);
    tried = true;
  }
  void* ctx = nullptr;
  if (fn == nullptr || fn(&ctx) != 0) return nullptr;
  return ctx;
}

// Device address of the scratch array on the current device; looked up once per device.
int static_scratch_base(unsigned char** base) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return gdn::set_error(B200GDN_ERR_CUDA, "chunk_fwd_static: cudaGetDevice: %s", cudaGetErrorString(e));
  if (dev < 0 || dev >= kMaxDevices)
    return gdn::set_error(B200GDN_ERR_UNSUPPORTED, "chunk_fwd_static: device index %d outside [0,%d)", dev, kMaxDevices);
  std::lock_guard<std::mutex> lock(g_scratch_mutex);
  void* ctx = current_context();
  if (g_scratch_addr[dev] == nullptr || g_scratch_ctx[dev] != ctx) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_static_scratch);
    if (e != cudaSuccess || p == nullptr)
      return gdn::set_error(B200GDN_ERR_CUDA, "chunk_fwd_static: cudaGetSymbolAddress on device %d: %s", dev,
                            cudaGetErrorString(e));
    g_scratch_addr[dev] = p;
    g_scratch_ctx[dev] = ctx;
  }
  *base = static_cast<unsigned char*>(g_scratch_addr[dev]);
  return 0;
}

inline size_t align256(size_t x) { return (x + 255) & ~static_cast<size_t>(255); }

}  // namespace

extern "C" int b200gdn_chunk_fwd_static(const b200gdn_chunk_args* a, void* stream) {
  using namespace gdn;
  const char* who = "chunk_fwd_static";
  reset_launch_count();
  if (a == nullptr) return set_error(B200GDN_ERR_BAD_ARGUMENT, "%s: args is NULL", who);
  if (a->struct_bytes != (int32_t)sizeof(b200gdn_chunk_args))
    return set_error(B200GDN_ERR_BAD_ARGUMENT, "%s: struct_bytes %d != %zu (ABI mismatch)", who, a->struct_bytes,
                     sizeof(b200gdn_chunk_args));
  if (a->rows <= 0 || a->H <= 0 || a->HV <= 0 || a->K <= 0 || a->V <= 0 || a->n_seq <= 0 || a->n_chunks <= 0 ||
      a->HV % a->H != 0)
    return set_error(B200GDN_ERR_BAD_ARGUMENT, "%s: bad sizes (rows=%d H=%d HV=%d K=%d V=%d n_seq=%d n_chunks=%d)", who,
                     a->rows, a->H, a->HV, a->K, a->V, a->n_seq, a->n_chunks);
  if (a->HV > 65535 || a->n_seq > 65535)
    return set_error(B200GDN_ERR_UNSUPPORTED, "%s: HV and n_seq are grid dimensions (<= 65535)", who);
  if (!a->chunk_meta || !a->seq_meta || !a->q || !a->k || !a->v || !a->g || !a->beta || !a->o)
    return set_error(B200GDN_ERR_BAD_ARGUMENT, "%s: q, k, v, g, beta, o and both chunk tables are required", who);

  // carve the array: gamma | A | qk | w | u, each region 256-byte aligned (h and v_new are only read by a backward
  // pass, which this entry point does not serve: the scan does not write them)
  const size_t rh = (size_t)a->rows * a->HV;
  const size_t sz_gamma = align256((size_t)a->n_chunks * a->HV * B200GDN_CHUNK * sizeof(float));
  const size_t sz_A = align256(rh * B200GDN_CHUNK * 2);
  const size_t sz_w = align256(rh * a->K * 2);
  const size_t sz_u = align256(rh * a->V * 2);
  const size_t need = sz_gamma + 2 * sz_A + sz_w + sz_u;
  if (need > (size_t)B200GDN_STATIC_SCRATCH_BYTES)
    return set_error(B200GDN_ERR_TOO_LARGE,
                     "%s: this problem needs %zu bytes of intermediates but the built-in array holds %zu; "
                     "use b200gdn_chunk_fwd with caller-allocated buffers, or split the batch",
                     who, need, (size_t)B200GDN_STATIC_SCRATCH_BYTES);

  unsigned char* base = nullptr;
  if (int e = static_scratch_base(&base)) return e;

  b200gdn_chunk_args b = *a;
  unsigned char* p = base;
  b.gamma = reinterpret_cast<float*>(p); p += sz_gamma;
  b.A = p; p += sz_A;
  b.qk = p; p += sz_A;
  b.w = p; p += sz_w;
  b.u = p;
  b.v_new = nullptr;
  b.h = nullptr;
  b.stage_mask = 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (int e = launch_intra_fwd(b, st)) return e;
  return launch_scan_out_fwd(b, st);
}
