// rswa_bwd_noalloc: the whole backward with its scratch memory inside the library.
//
// Who this is for.  rswa_bwd needs scratch memory next to its inputs and outputs (two fp32 rows per
// batch row and head: delta = rowsum(dO * O) and the scaled log-sum-exp, written by a small kernel
// and read by both tensor-core kernels), and leaves it to the caller to allocate it.  Some
// callers cannot do that at the point where they call us: a plugin that runs inside another
// runtime's execution phase and is only handed the tensors of the operator, a
// serving process whose device memory was carved up completely at start-up, code that is not
// allowed to call cudaMalloc because that call synchronises the whole device and would stall the
// other streams of the process.  For them the scratch lives in a fixed array in this library's
// device image; the caller passes inputs and outputs only.
//
// The price: the array has a fixed size (RSWA_NOALLOC_SCRATCH_BYTES, 64 MiB + 256 bytes) that every GPU which
// loads the library holds until the process exits, problems that need more are rejected, and all
// calls share the one array, so two calls that may overlap on the GPU (different streams) race.
#include <mutex>

#include "rswa_common.cuh"

namespace {

// File-scope device array.  In host code this name is only a handle for the runtime; the address
// the kernels must be given comes from cudaGetSymbolAddress, asked for once per device.
static __device__ __align__(256) unsigned char g_noalloc_scratch[RSWA_NOALLOC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
std::mutex g_setup_mutex;
void* g_scratch_addr[kMaxDevices] = {nullptr};

// Address of the scratch array on the current device; resolved on the first call for that device.
int scratch_for_current_device(void** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) {
    rswa::set_error("rswa_bwd_noalloc: cudaGetDevice: %s", cudaGetErrorString(e));
    return RSWA_E_CUDA;
  }
  if (dev < 0 || dev >= kMaxDevices) {
    rswa::set_error("rswa_bwd_noalloc: device index %d is outside the %d devices this entry point keeps a scratch address for",
                    dev, kMaxDevices);
    return RSWA_E_UNSUPPORTED;
  }
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (g_scratch_addr[dev] == nullptr) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
    if (e != cudaSuccess || ptr == nullptr) {
      rswa::set_error("rswa_bwd_noalloc: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
      return RSWA_E_CUDA;
    }
    g_scratch_addr[dev] = ptr;
  }
  *out = g_scratch_addr[dev];
  return RSWA_OK;
}

}  // namespace

extern "C" int64_t rswa_noalloc_scratch_bytes(void) { return RSWA_NOALLOC_SCRATCH_BYTES; }

extern "C" int rswa_bwd_noalloc(const rswa_bwd_params_t* p, void* stream) {
  if (p == nullptr) {
    rswa::set_error("rswa_bwd_noalloc: null params");
    return RSWA_E_ARG;
  }
  const int64_t need = rswa_bwd_workspace_bytes(p->g.batch, p->g.q_len, p->g.n_q_heads, p->g.head_dim);
  if (need < 0) {
    rswa::set_error("rswa_bwd_noalloc: unsupported shape (batch %d, q_len %d, heads %d, head_dim %d)", p->g.batch,
                    p->g.q_len, p->g.n_q_heads, p->g.head_dim);
    return RSWA_E_UNSUPPORTED;
  }
  if (need > RSWA_NOALLOC_SCRATCH_BYTES) {
    rswa::set_error(
        "rswa_bwd_noalloc: this problem needs %lld bytes of scratch, the built-in array holds %lld "
        "(batch * n_q_heads * q_len, padded to whole tiles, may be %lld at most); use rswa_bwd with a caller-owned workspace",
        static_cast<long long>(need), static_cast<long long>(RSWA_NOALLOC_SCRATCH_BYTES),
        static_cast<long long>((RSWA_NOALLOC_SCRATCH_BYTES - 256) / 8));
    return RSWA_E_NOALLOC_SIZE;
  }
  // the remaining argument checks come before the array is looked up: a rejected call touches nothing
  int rc = rswa::check_geom(p->g, false);
  if (rc) return rc;
  void* scratch = nullptr;
  rc = scratch_for_current_device(&scratch);
  if (rc) return rc;
  // Same work as rswa_bwd over the built-in scratch.  A whole backward in one call: INIT rewrites the
  // delta and scaled-lse rows (the array still holds the previous call's), FINISH produces dq.
  rswa_bwd_params_t q = *p;
  q.workspace = scratch;
  q.workspace_bytes = RSWA_NOALLOC_SCRATCH_BYTES;
  q.flags = RSWA_BWD_INIT | RSWA_BWD_FINISH;
  return rswa_bwd(&q, stream);
}
