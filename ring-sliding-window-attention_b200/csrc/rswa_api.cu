// C-ABI layer: argument checks, TMA descriptor set-up, launches.  See include/rswa.h.
#include <cstdarg>
#include <cstdio>
#include <cstring>

#include "rswa_common.cuh"

namespace rswa {

int launch_fwd(const FwdKernelParams& kp, int dtype, cudaStream_t stream);
int launch_bwd(const BwdKernelParams& kp, int dtype, int total_key_tiles, cudaStream_t stream);
int launch_delta(const rswa_bwd_params_t& p, float* delta, float* lse2, int q_len_pad, cudaStream_t stream);
int launch_dq(const BwdKernelParams& kp, int dtype, cudaStream_t stream);

static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode() {
  static EncodeTiledFn fn = nullptr;
  if (fn) return fn;
  void* sym = nullptr;
  cudaDriverEntryPointQueryResult qres;
  cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres);
  if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess || sym == nullptr) {
    set_error("cuTensorMapEncodeTiled not available: %s", cudaGetErrorString(e));
    return nullptr;
  }
  fn = reinterpret_cast<EncodeTiledFn>(sym);
  return fn;
}

// Encoded maps are kept in a small per-thread cache keyed by everything the encoding depends on: a
// training step presents the same few tensors (same pointers from a caching allocator, same shapes) call
// after call, and each encoding is a driver call of a microsecond or two, a dozen of them per step and rank.
namespace {
struct MapKey {
  const void* base;
  int dtype, batch, tokens, heads;
  long long sb, st, sh;
  bool operator==(const MapKey& o) const {
    return base == o.base && dtype == o.dtype && batch == o.batch && tokens == o.tokens && heads == o.heads &&
           sb == o.sb && st == o.st && sh == o.sh;
  }
};
constexpr int kMapCacheSize = 64;
struct MapCache {
  MapKey key[kMapCacheSize];
  CUtensorMap map[kMapCacheSize];
  int used = 0, next = 0;
};
thread_local MapCache t_map_cache;
}  // namespace

int make_tile_map(CUtensorMap* map, const void* base, int dtype, int batch, int tokens, int heads,
                  long long sb, long long st, long long sh) {
  EncodeTiledFn enc = get_encode();
  if (!enc) return RSWA_E_CUDA;
  // The encoder is a driver entry point and wants a context current on the calling thread.  A thread
  // that has made no runtime call yet (an autograd worker calling the backward first) may have none:
  // once per thread, bind the primary context of the thread's current device.  (Once, because the
  // call synchronises and must not recur inside a stream capture.)
  static thread_local bool t_context_bound = false;
  if (!t_context_bound) {
    cudaFree(nullptr);
    t_context_bound = true;
  }
  if (base == nullptr || (reinterpret_cast<uintptr_t>(base) & 15) != 0) {
    set_error("tensor base pointer must be non-null and 16-byte aligned");
    return RSWA_E_ARG;
  }
  if (tokens <= 0 || heads <= 0 || batch <= 0) {
    set_error("tensor extents must be positive (batch %d, tokens %d, heads %d)", batch, tokens, heads);
    return RSWA_E_ARG;
  }
  if ((sb % 8) != 0 || (st % 8) != 0 || (sh % 8) != 0 || st <= 0 || sh <= 0 || sb < 0) {
    set_error("tensor strides must be positive multiples of 8 elements (got %lld, %lld, %lld)", sb, st, sh);
    return RSWA_E_ARG;
  }
  if (batch == 1 && sb == 0) sb = static_cast<long long>(tokens) * st;
  const MapKey key{base, dtype, batch, tokens, heads, sb, st, sh};
  MapCache& cache = t_map_cache;
  for (int i = 0; i < cache.used; ++i) {
    if (cache.key[i] == key) {
      *map = cache.map[i];
      return RSWA_OK;
    }
  }
  cuuint64_t dims[4] = {static_cast<cuuint64_t>(kHeadDim), static_cast<cuuint64_t>(heads),
                        static_cast<cuuint64_t>(tokens), static_cast<cuuint64_t>(batch)};
  cuuint64_t strides[3] = {static_cast<cuuint64_t>(sh) * 2, static_cast<cuuint64_t>(st) * 2,
                           static_cast<cuuint64_t>(sb) * 2};
  cuuint32_t box[4] = {64, 1, static_cast<cuuint32_t>(kTile), 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = enc(map, dtype == RSWA_DTYPE_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                   4, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled failed with code %d (tokens %d heads %d strides %lld %lld %lld)",
              static_cast<int>(r), tokens, heads, sb, st, sh);
    return RSWA_E_CUDA;
  }
  const int slot = cache.used < kMapCacheSize ? cache.used++ : (cache.next++ % kMapCacheSize);
  cache.key[slot] = key;
  cache.map[slot] = *map;
  return RSWA_OK;
}

int check_geom(const rswa_geom_t& g, bool need_grads) {
  if (g.dtype != RSWA_DTYPE_BF16 && g.dtype != RSWA_DTYPE_FP16) {
    set_error("dtype must be bf16 (0) or fp16 (1), got %d", g.dtype);
    return RSWA_E_UNSUPPORTED;
  }
  if (g.head_dim != kHeadDim) {
    set_error("head_dim must be %d, got %d", kHeadDim, g.head_dim);
    return RSWA_E_UNSUPPORTED;
  }
  if (g.batch <= 0 || g.q_len <= 0 || g.n_q_heads <= 0 || g.n_kv_heads <= 0) {
    set_error("batch, q_len and head counts must be positive");
    return RSWA_E_ARG;
  }
  if (g.n_q_heads % g.n_kv_heads != 0) {
    set_error("Number of query heads must be divisible by number of key/value heads");
    return RSWA_E_ARG;
  }
  if (g.window < 0 || g.n_sink < 0 || g.q_pos_start < 0) {
    set_error("window, n_sink and q_pos_start must be non-negative");
    return RSWA_E_ARG;
  }
  if (!(g.softmax_scale > 0.f)) {
    set_error("softmax_scale must be positive");
    return RSWA_E_ARG;
  }
  if (g.cu_seqlens != nullptr && (g.batch != 1 || g.n_seqs <= 0)) {
    set_error("packed (cu_seqlens) input needs batch == 1 and n_seqs > 0");
    return RSWA_E_ARG;
  }
  if (g.n_spans < 0 || g.n_spans > RSWA_MAX_SPANS) {
    set_error("n_spans must be in [0, %d]", RSWA_MAX_SPANS);
    return RSWA_E_ARG;
  }
  if (static_cast<long long>(g.q_pos_start) + g.q_len + g.window >= 0x7fffffffLL) {
    set_error("positions overflow int32");
    return RSWA_E_ARG;
  }
  for (int i = 0; i < g.n_spans; ++i) {
    const rswa_span_t& s = g.spans[i];
    if (s.len <= 0 || s.pos_start < 0 || s.k == nullptr || s.v == nullptr) {
      set_error("span %d: needs k, v, len > 0 and pos_start >= 0", i);
      return RSWA_E_ARG;
    }
    if (need_grads && (s.dk == nullptr || s.dv == nullptr)) {
      set_error("span %d: dk and dv are required in backward", i);
      return RSWA_E_ARG;
    }
    for (int j = 0; j < i; ++j) {
      const rswa_span_t& o = g.spans[j];
      if (s.pos_start < o.pos_start + o.len && o.pos_start < s.pos_start + s.len) {
        set_error("spans %d and %d overlap in position", j, i);
        return RSWA_E_ARG;
      }
    }
  }
  return RSWA_OK;
}

static int fill_span_maps(const rswa_geom_t& g, CUtensorMap* kmaps, CUtensorMap* vmaps, int* pos, int* len) {
  for (int i = 0; i < g.n_spans; ++i) {
    const rswa_span_t& s = g.spans[i];
    int rc = make_tile_map(&kmaps[i], s.k, g.dtype, g.batch, s.len, g.n_kv_heads, s.kv_stride_b, s.kv_stride_t,
                           s.kv_stride_h);
    if (rc) return rc;
    rc = make_tile_map(&vmaps[i], s.v, g.dtype, g.batch, s.len, g.n_kv_heads, s.kv_stride_b, s.kv_stride_t,
                       s.kv_stride_h);
    if (rc) return rc;
    pos[i] = s.pos_start;
    len[i] = s.len;
  }
  return RSWA_OK;
}

int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace rswa

using namespace rswa;

extern "C" int rswa_abi_version(void) { return RSWA_ABI_VERSION; }
extern "C" const char* rswa_last_error(void) { return g_err; }

extern "C" int rswa_fwd(const rswa_fwd_params_t* p, void* stream) {
  if (p == nullptr) {
    set_error("rswa_fwd: null params");
    return RSWA_E_ARG;
  }
  const rswa_geom_t& g = p->g;
  int rc = check_geom(g, false);
  if (rc) return rc;
  if (p->q == nullptr || p->out == nullptr || p->lse == nullptr || p->status == nullptr) {
    set_error("rswa_fwd: q, out, lse and status are required");
    return RSWA_E_ARG;
  }
  if (!aligned16(p->out) || (p->o_stride_b % 8) || (p->o_stride_t % 8) || (p->o_stride_h % 8)) {
    set_error("rswa_fwd: out must be 16-byte aligned with strides that are multiples of 8 elements");
    return RSWA_E_ARG;
  }
  const int n_tiles_all = (g.q_len + kTile - 1) / kTile;
  int qb = p->q_tile_begin, qe = p->q_tile_end <= 0 ? n_tiles_all : p->q_tile_end;
  if (qb < 0 || qe > n_tiles_all || qb > qe) {
    set_error("rswa_fwd: query tile range [%d, %d) outside [0, %d]", qb, qe, n_tiles_all);
    return RSWA_E_ARG;
  }
  FwdKernelParams kp;
  memset(&kp, 0, sizeof(kp));
  rc = make_tile_map(&kp.q_map, p->q, g.dtype, g.batch, g.q_len, g.n_q_heads, p->q_stride_b, p->q_stride_t,
                     p->q_stride_h);
  if (rc) return rc;
  rc = fill_span_maps(g, kp.k_map, kp.v_map, kp.span_pos, kp.span_len);
  if (rc) return rc;
  kp.n_spans = g.n_spans;
  kp.batch = g.batch;
  kp.q_len = g.q_len;
  kp.hq = g.n_q_heads;
  kp.hkv = g.n_kv_heads;
  kp.q_pos_start = g.q_pos_start;
  kp.window = g.window;
  kp.n_sink = g.n_sink;
  kp.scale_log2 = g.softmax_scale * 1.4426950408889634f;
  kp.cu = g.cu_seqlens;
  kp.n_seqs = g.n_seqs;
  kp.out = p->out;
  kp.o_sb = p->o_stride_b;
  kp.o_st = p->o_stride_t;
  kp.o_sh = p->o_stride_h;
  kp.lse = p->lse;
  kp.l_sb = p->lse_stride_b;
  kp.l_sh = p->lse_stride_h;
  kp.q_tile_begin = qb;
  kp.n_q_tiles = qe - qb;
  kp.carry = p->carry != 0;
  kp.status = p->status;
  return launch_fwd(kp, g.dtype, static_cast<cudaStream_t>(stream));
}

extern "C" int64_t rswa_bwd_workspace_bytes(int32_t batch, int32_t q_len, int32_t n_q_heads, int32_t head_dim) {
  if (batch <= 0 || q_len <= 0 || n_q_heads <= 0 || head_dim != kHeadDim) return -1;
  const int64_t q_len_pad = (static_cast<int64_t>(q_len) + kTile - 1) / kTile * kTile;
  // two fp32 rows per (batch, head): delta = rowsum(dO * O) and lse * log2(e), padded to whole tiles;
  // then 256 bytes that hold the work counters of the dQ and dK/dV kernels
  return 2 * static_cast<int64_t>(batch) * n_q_heads * q_len_pad * 4 + 256;
}

extern "C" int rswa_bwd(const rswa_bwd_params_t* p, void* stream_) {
  if (p == nullptr) {
    set_error("rswa_bwd: null params");
    return RSWA_E_ARG;
  }
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const rswa_geom_t& g = p->g;
  int rc = check_geom(g, false);
  if (rc) return rc;
  if (!p->q || !p->out || !p->dout || !p->lse || !p->workspace || !p->status) {
    set_error("rswa_bwd: q, out, dout, lse, workspace and status are required");
    return RSWA_E_ARG;
  }
  const bool want_dq = (p->flags & RSWA_BWD_FINISH) != 0;
  if (want_dq && !p->dq) {
    set_error("rswa_bwd: dq is required with RSWA_BWD_FINISH");
    return RSWA_E_ARG;
  }
  const int64_t need = rswa_bwd_workspace_bytes(g.batch, g.q_len, g.n_q_heads, g.head_dim);
  if (p->workspace_bytes < need || (reinterpret_cast<uintptr_t>(p->workspace) & 255) != 0) {
    set_error("rswa_bwd: workspace needs %lld bytes, 256-byte aligned (got %lld)", (long long)need,
              (long long)p->workspace_bytes);
    return RSWA_E_ARG;
  }
  if ((want_dq && (!aligned16(p->dq) || (p->dq_stride_b % 8) || (p->dq_stride_t % 8) || (p->dq_stride_h % 8))) ||
      !aligned16(p->out) || (p->o_stride_t % 8) || (p->o_stride_h % 8) || (p->o_stride_b % 8)) {
    set_error("rswa_bwd: dq/out must be 16-byte aligned with strides that are multiples of 8 elements");
    return RSWA_E_ARG;
  }
  const int q_len_pad = (g.q_len + kTile - 1) / kTile * kTile;
  float* delta = static_cast<float*>(p->workspace);
  float* lse2 = delta + static_cast<int64_t>(g.batch) * g.n_q_heads * q_len_pad;
  int* dq_counter = reinterpret_cast<int*>(lse2 + static_cast<int64_t>(g.batch) * g.n_q_heads * q_len_pad);
  {  // both work counters, ahead of every kernel of this call, so that the reset sits in no timed interval
    cudaError_t e = cudaMemsetAsync(dq_counter, 0, 2 * sizeof(int), static_cast<cudaStream_t>(stream_));
    if (e != cudaSuccess) {
      set_error("rswa_bwd: cudaMemsetAsync: %s", cudaGetErrorString(e));
      return RSWA_E_CUDA;
    }
  }

  // kq: every span (the dQ kernel sums over all keys); kk: only the spans whose dK/dV are wanted
  BwdKernelParams kq, kk;
  memset(&kq, 0, sizeof(kq));
  rc = make_tile_map(&kq.q_map, p->q, g.dtype, g.batch, g.q_len, g.n_q_heads, p->q_stride_b, p->q_stride_t,
                     p->q_stride_h);
  if (rc) return rc;
  rc = make_tile_map(&kq.do_map, p->dout, g.dtype, g.batch, g.q_len, g.n_q_heads, p->do_stride_b,
                     p->do_stride_t, p->do_stride_h);
  if (rc) return rc;
  rc = fill_span_maps(g, kq.k_map, kq.v_map, kq.span_pos, kq.span_len);
  if (rc) return rc;
  kq.n_spans = g.n_spans;
  kq.batch = g.batch;
  kq.q_len = g.q_len;
  kq.hq = g.n_q_heads;
  kq.hkv = g.n_kv_heads;
  kq.q_pos_start = g.q_pos_start;
  kq.window = g.window;
  kq.n_sink = g.n_sink;
  kq.scale = g.softmax_scale;
  kq.scale_log2 = g.softmax_scale * 1.4426950408889634f;
  kq.cu = g.cu_seqlens;
  kq.n_seqs = g.n_seqs;
  kq.lse2 = lse2;
  kq.delta = delta;
  kq.d_sb = static_cast<long long>(g.n_q_heads) * q_len_pad;
  kq.d_sh = q_len_pad;
  kq.dq = p->dq;
  kq.dq_sb = p->dq_stride_b;
  kq.dq_st = p->dq_stride_t;
  kq.dq_sh = p->dq_stride_h;
  kq.status = p->status;

  kk = kq;
  int n_k = 0, total_tiles = 0;
  for (int i = 0; i < g.n_spans; ++i) {
    const rswa_span_t& s = g.spans[i];
    if (s.dk == nullptr && s.dv == nullptr) continue;  // no gradients wanted for this span in this call
    if (s.dk == nullptr || s.dv == nullptr) {
      set_error("rswa_bwd: span %d: dk and dv must be given together", i);
      return RSWA_E_ARG;
    }
    const int al = s.grad_fp32 ? 4 : 8;
    if (!aligned16(s.dk) || !aligned16(s.dv) || (s.dkv_stride_b % al) || (s.dkv_stride_t % al) ||
        (s.dkv_stride_h % al)) {
      set_error("rswa_bwd: span %d dk/dv must be 16-byte aligned with 16-byte multiple strides", i);
      return RSWA_E_ARG;
    }
    kk.k_map[n_k] = kq.k_map[i];
    kk.v_map[n_k] = kq.v_map[i];
    kk.span_pos[n_k] = s.pos_start;
    kk.span_len[n_k] = s.len;
    kk.span_tile0[n_k] = total_tiles;
    total_tiles += (s.len + kTile - 1) / kTile;
    kk.dk[n_k] = s.dk;
    kk.dv[n_k] = s.dv;
    kk.dkv_sb[n_k] = s.dkv_stride_b;
    kk.dkv_st[n_k] = s.dkv_stride_t;
    kk.dkv_sh[n_k] = s.dkv_stride_h;
    kk.grad_fp32[n_k] = s.grad_fp32;
    ++n_k;
  }
  kk.span_tile0[n_k] = total_tiles;
  kk.n_spans = n_k;

  if (p->flags & RSWA_BWD_INIT) {
    rc = launch_delta(*p, delta, lse2, q_len_pad, stream);
    if (rc) return rc;
  }
  if (p->ev_main_start) cudaEventRecord(static_cast<cudaEvent_t>(p->ev_main_start), stream);
  if (total_tiles > 0) {
    kk.dkv_counter = dq_counter + 1;
    rc = launch_bwd(kk, g.dtype, total_tiles, stream);
    if (rc) return rc;
  }
  if (p->ev_main_mid) cudaEventRecord(static_cast<cudaEvent_t>(p->ev_main_mid), stream);
  if (want_dq) {
    kq.dq_counter = dq_counter;
    rc = launch_dq(kq, g.dtype, stream);
    if (rc) return rc;
  }
  if (p->ev_main_stop) cudaEventRecord(static_cast<cudaEvent_t>(p->ev_main_stop), stream);
  return RSWA_OK;
}

extern "C" void* rswa_event_create(void) {
  cudaEvent_t ev = nullptr;
  if (cudaEventCreate(&ev) != cudaSuccess) {
    set_error("rswa_event_create: cudaEventCreate failed");
    return nullptr;
  }
  return ev;
}
extern "C" void rswa_event_destroy(void* ev) {
  if (ev) cudaEventDestroy(static_cast<cudaEvent_t>(ev));
}
extern "C" int rswa_event_record(void* ev, void* stream) {
  if (!ev || cudaEventRecord(static_cast<cudaEvent_t>(ev), static_cast<cudaStream_t>(stream)) != cudaSuccess) {
    set_error("rswa_event_record failed");
    return RSWA_E_CUDA;
  }
  return RSWA_OK;
}
extern "C" int rswa_event_wait(void* ev, void* stream) {
  if (!ev || cudaStreamWaitEvent(static_cast<cudaStream_t>(stream), static_cast<cudaEvent_t>(ev), 0) != cudaSuccess) {
    set_error("rswa_event_wait failed");
    return RSWA_E_CUDA;
  }
  return RSWA_OK;
}
extern "C" float rswa_event_elapsed_ms(void* start, void* stop) {
  float ms = -1.f;
  if (!start || !stop) return -1.f;
  if (cudaEventSynchronize(static_cast<cudaEvent_t>(stop)) != cudaSuccess) return -1.f;
  if (cudaEventElapsedTime(&ms, static_cast<cudaEvent_t>(start), static_cast<cudaEvent_t>(stop)) != cudaSuccess) return -1.f;
  return ms;
}
