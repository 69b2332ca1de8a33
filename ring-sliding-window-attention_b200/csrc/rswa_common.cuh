// Internal declarations shared by the kernels and the C-ABI layer.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/rswa.h"

namespace rswa {

constexpr int kTile = RSWA_TILE;       // rows of a query tile and of a key tile
constexpr int kHeadDim = 128;
constexpr int kBoxBytes = 16384;       // one TMA box: 128 rows x 64 x 16-bit, 128-byte swizzle
constexpr int kTileBytes = 2 * kBoxBytes;
constexpr int kMaxEntries = 2 * RSWA_MAX_SPANS;

// device-side error codes written to the status word
enum : int {
  kErrWaitProducer = 101,
  kErrWaitMma = 102,
  kErrWaitSoftmax = 103,
  kErrWaitEpilogue = 104,
};

struct FwdKernelParams {
  CUtensorMap q_map;
  CUtensorMap k_map[RSWA_MAX_SPANS];
  CUtensorMap v_map[RSWA_MAX_SPANS];
  int span_pos[RSWA_MAX_SPANS];
  int span_len[RSWA_MAX_SPANS];
  int n_spans;
  int batch, q_len, hq, hkv;
  int q_pos_start, window, n_sink;
  float scale_log2;  // softmax_scale * log2(e)
  const int* cu;
  int n_seqs;
  void* out;
  long long o_sb, o_st, o_sh;
  float* lse;
  long long l_sb, l_sh;
  int q_tile_begin, n_q_tiles;
  int carry;  // out / lse hold a partial result over other keys: continue it instead of starting over
  int* status;
};

struct BwdKernelParams {
  CUtensorMap q_map;
  CUtensorMap do_map;
  CUtensorMap k_map[RSWA_MAX_SPANS];
  CUtensorMap v_map[RSWA_MAX_SPANS];
  int span_pos[RSWA_MAX_SPANS];
  int span_len[RSWA_MAX_SPANS];
  int span_tile0[RSWA_MAX_SPANS + 1];  // prefix sum of key tiles per span
  void* dk[RSWA_MAX_SPANS];
  void* dv[RSWA_MAX_SPANS];
  long long dkv_sb[RSWA_MAX_SPANS], dkv_st[RSWA_MAX_SPANS], dkv_sh[RSWA_MAX_SPANS];
  int grad_fp32[RSWA_MAX_SPANS];
  int n_spans;
  int batch, q_len, hq, hkv;
  int q_pos_start, window, n_sink;
  float scale_log2;
  float scale;
  const int* cu;
  int n_seqs;
  // rows prepared by the delta kernel, both [batch, hq, q_len_pad] fp32, 512-byte aligned per
  // 128-query tile and both NEGATED: -lse * log2(e) (-inf past q_len) and -delta = -rowsum(dO * O)
  // (0 past q_len)
  const float* lse2;
  const float* delta;
  long long d_sb, d_sh;
  void* dq;  // [batch, q_len, hq, 128], 16-bit, written by the dQ kernel
  int* dq_counter;   // work counter of the dQ kernel, zeroed before its launch
  int* dkv_counter;  // work counter of the dK/dV kernel, likewise
  long long dq_sb, dq_st, dq_sh;
  int* status;
};

// Sequence [start, end) containing global position p.  cu has n_seqs + 1 entries.
__device__ __forceinline__ void seq_of(const int* __restrict__ cu, int n_seqs, int p, int& start,
                                       int& end) {
  if (cu == nullptr) {
    start = 0;
    end = 0x7fffffff;
    return;
  }
  int lo = 0, hi = n_seqs;
  while (lo < hi) {
    int mid = (lo + hi + 1) >> 1;
    if (__ldg(cu + mid) <= p) lo = mid; else hi = mid - 1;
  }
  start = __ldg(cu + lo);
  end = (lo < n_seqs) ? __ldg(cu + lo + 1) : 0x7fffffff;
}

// Optional in-kernel timeline (development builds only, -DRSWA_TRACE): one chosen CTA stamps clock64()
// into a per-file device array that a small extern "C" reader copies out.  Compiles to nothing otherwise.
#ifdef RSWA_TRACE
#ifndef RSWA_TRACE_CTA
#define RSWA_TRACE_CTA 2000
#endif
#define RSWA_TRACE_SLOTS 2048
#define RSWA_TRACE_DECL(name)                                                                    \
  static __device__ long long g_trace_##name[RSWA_TRACE_SLOTS];                                  \
  extern "C" int rswa_trace_read_##name(long long* out) {                                         \
    return static_cast<int>(cudaMemcpyFromSymbol(out, g_trace_##name, sizeof(g_trace_##name)));  \
  }
#define RSWA_TRC(name, cond, slot)                                                               \
  do {                                                                                           \
    if (blockIdx.x == RSWA_TRACE_CTA && (cond) && (slot) < RSWA_TRACE_SLOTS) g_trace_##name[slot] = clock64(); \
  } while (0)
#else
#define RSWA_TRACE_DECL(name)
#define RSWA_TRC(name, cond, slot) do { } while (0)
#endif

// host side -------------------------------------------------------------------------------
void set_error(const char* fmt, ...);
// 4-D map over a [batch, tokens, heads, 128] 16-bit tensor (strides in elements), box = 64
// elements x 1 head x 128 tokens x 1 batch, 128-byte swizzle, zero fill out of bounds.
int make_tile_map(CUtensorMap* map, const void* base, int dtype, int batch, int tokens, int heads,
                  long long sb, long long st, long long sh);
int check_geom(const rswa_geom_t& g, bool need_grads);
int sm_count();  // SMs of the current device (cached per device)

}  // namespace rswa
