// Bandwidth-bound helpers around the attention kernels: delta = rowsum(dO * O) and scaled lse rows,
// the log-sum-exp merge of two partial results, halo-gradient accumulation and the final cast.
// All are straight streaming kernels: 16-byte accesses, one warp per 128-element row where rows
// are involved, grid sized from the data.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "rswa_common.cuh"

namespace rswa {
namespace {

template <bool kBf16>
__device__ __forceinline__ float2 unpack2(uint32_t w) {
  if constexpr (kBf16) {
    return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
  } else {
    __half2 h = *reinterpret_cast<__half2*>(&w);
    return __half22float2(h);
  }
}
template <bool kBf16>
__device__ __forceinline__ uint32_t pack2f(float lo, float hi) {
  if constexpr (kBf16) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  } else {
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  }
}

// A warp takes 32 consecutive tokens of one (batch row, head): half a warp per 128-element row (16 bytes
// per lane and tensor), eight rows in flight per lane pair, and the 32 results leave as ONE 128-byte
// segment of each output row (one token per lane) instead of 32 scattered words.  Writes
// -delta = -rowsum(dO * O) and -lse2 = -lse * log2(e) into rows padded to whole 128-query tiles; the
// padding gets -delta = 0 and -lse2 = -inf so that P = exp2(s - lse2) vanishes there.
template <bool kBf16>
__global__ void delta_kernel(const uint16_t* __restrict__ out, long long o_sb, long long o_st, long long o_sh,
                             const uint16_t* __restrict__ dout, long long d_sb, long long d_st, long long d_sh,
                             const float* __restrict__ lse, long long l_sb, long long l_sh,
                             float* __restrict__ delta, float* __restrict__ lse2, int batch, int q_len, int hq,
                             int q_len_pad) {
  const long long wid = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;  // warp task
  const int lane = threadIdx.x & 31;
  const int sub = lane & 15, hi = lane >> 4;
  const int t_blocks = q_len_pad >> 5;  // q_len_pad is a multiple of 128
  const long long n_tasks = static_cast<long long>(batch) * hq * t_blocks;
  if (wid >= n_tasks) return;
  const int tb = wid % t_blocks;       // token block fastest: neighbouring warps read neighbouring tokens
  const long long bh = wid / t_blocks;
  const int h = bh % hq;
  const int b = bh / hq;
  const int t0 = tb * 32;
  const uint16_t* po = out + b * o_sb + h * o_sh + sub * 8;
  const uint16_t* pd = dout + b * d_sb + h * d_sh + sub * 8;
  float mine = 0.f;  // the sum of the token this lane will write (t0 + lane)
#pragma unroll
  for (int blk = 0; blk < 2; ++blk) {  // 16 tokens per block: 8 loads of each tensor in flight per lane
    uint4 a[8], d[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int t = t0 + blk * 16 + 2 * i + hi;
      if (t < q_len) {
        a[i] = *reinterpret_cast<const uint4*>(po + t * o_st);
        d[i] = *reinterpret_cast<const uint4*>(pd + t * d_st);
      } else {
        a[i] = make_uint4(0, 0, 0, 0);
        d[i] = make_uint4(0, 0, 0, 0);
      }
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const uint32_t aw[4] = {a[i].x, a[i].y, a[i].z, a[i].w}, dw[4] = {d[i].x, d[i].y, d[i].z, d[i].w};
      float s = 0.f;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 x = unpack2<kBf16>(aw[j]), y = unpack2<kBf16>(dw[j]);
        s += x.x * y.x + x.y * y.y;
      }
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
      // lanes 0-15 hold the sum of token t0 + 16 blk + 2 i, lanes 16-31 that of the next one
      const float lo_sum = __shfl_sync(0xffffffffu, s, 0), hi_sum = __shfl_sync(0xffffffffu, s, 16);
      if (lane == blk * 16 + 2 * i) mine = lo_sum;
      if (lane == blk * 16 + 2 * i + 1) mine = hi_sum;
    }
  }
  const int t = t0 + lane;
  const long long idx = (static_cast<long long>(b) * hq + h) * q_len_pad + t;
  // both rows are stored NEGATED: the backward kernels only ever add them (s * scale - lse2, dP - delta),
  // once per score, and their inner loops are bound by instruction count
  delta[idx] = -mine;
  // (a row that saw no key at all has lse = -inf: it gets -inf like the padding, so that its P vanishes
  // whatever its scores are, -inf included, instead of turning into inf - inf)
  const float l = t < q_len ? lse[b * l_sb + h * l_sh + t] : -INFINITY;
  lse2[idx] = l > -INFINITY ? l * -1.4426950408889634f : -INFINITY;
}

// LSE merge.  A warp takes 32 consecutive tokens of one (batch row, head): lane i reads the two lse values
// of token i (one 128-byte segment each), forms the weights and writes the merged lse (one segment); the
// rows go through half a warp each (16 bytes per lane and tensor), eight rows of each input in flight
// per lane pair, their weights fetched from the owning lane with a shuffle.  In place (o == o_a) is allowed:
// a row is read and written by the same lanes.
template <bool kBf16>
__global__ void merge_kernel(const rswa_merge_params_t p, long long n_tasks) {
  const long long wid = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  if (wid >= n_tasks) return;
  const int lane = threadIdx.x & 31;
  const int sub = lane & 15, hi = lane >> 4;
  const int t_blocks = (p.q_len + 31) >> 5;
  const int tb = wid % t_blocks;
  const long long bh = wid / t_blocks;
  const int h = bh % p.n_heads;
  const long long b = bh / p.n_heads;
  const int t0 = tb * 32;
  const int tl = t0 + lane;
  const long long li = b * p.lse_stride_b + h * p.lse_stride_h + tl;
  float wa = 0.f, wb = 0.f, l = -INFINITY;
  if (tl < p.q_len) {
    const float la = p.lse_a[li], lb = p.lse_b[li];
    const float mx = fmaxf(la, lb);
    if (mx != -INFINITY) {
      const float ea = __expf(la - mx), eb = __expf(lb - mx);
      const float inv = 1.f / (ea + eb);
      wa = ea * inv;
      wb = eb * inv;
      l = mx + __logf(ea + eb);
    }
  }
  const uint16_t* pa = static_cast<const uint16_t*>(p.o_a) + b * p.oa_stride_b + h * p.oa_stride_h + sub * 8;
  const uint16_t* pb = static_cast<const uint16_t*>(p.o_b) + b * p.ob_stride_b + h * p.ob_stride_h + sub * 8;
  uint16_t* po = static_cast<uint16_t*>(p.o) + b * p.o_stride_b + h * p.o_stride_h + sub * 8;
#pragma unroll
  for (int blk = 0; blk < 2; ++blk) {
    uint4 va[8], vb[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int t = t0 + blk * 16 + 2 * i + hi;
      if (t < p.q_len) {
        va[i] = *reinterpret_cast<const uint4*>(pa + t * p.oa_stride_t);
        vb[i] = *reinterpret_cast<const uint4*>(pb + t * p.ob_stride_t);
      } else {
        va[i] = make_uint4(0, 0, 0, 0);
        vb[i] = make_uint4(0, 0, 0, 0);
      }
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int src = blk * 16 + 2 * i + hi;  // the lane that owns this row's token
      const float xa = __shfl_sync(0xffffffffu, wa, src), xb = __shfl_sync(0xffffffffu, wb, src);
      const uint32_t aw[4] = {va[i].x, va[i].y, va[i].z, va[i].w}, bw[4] = {vb[i].x, vb[i].y, vb[i].z, vb[i].w};
      uint32_t ow[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 fa = unpack2<kBf16>(aw[k]), fb = unpack2<kBf16>(bw[k]);
        ow[k] = pack2f<kBf16>(fa.x * xa + fb.x * xb, fa.y * xa + fb.y * xb);
      }
      const int t = t0 + src;
      if (t < p.q_len) *reinterpret_cast<uint4*>(po + t * p.o_stride_t) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
    }
  }
  if (tl < p.q_len) p.lse[li] = l;
}

// In-place merge into a float accumulator (and a float or double lse), the precision the reference
// carries between ring hops.  One warp per (b, t, h) row, 4 elements per lane and pass.
// kind of the incoming output: 0 bf16, 1 fp16, 2 float.
template <int kKind, typename LseT>
__global__ void merge_acc_kernel(const rswa_merge_acc_params_t p, long long n_rows) {
  const long long row = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (row >= n_rows) return;
  const int h = row % p.n_heads;
  const long long bt = row / p.n_heads;
  const int t = bt % p.q_len;
  const long long b = bt / p.q_len;
  LseT* la_ptr = static_cast<LseT*>(p.acc_lse) + b * p.acc_lse_stride_b + h * p.acc_lse_stride_h + t;
  const float la = static_cast<float>(*la_ptr);  // the reference's kernel also reads the double as float
  const float lb = p.new_lse[b * p.new_lse_stride_b + h * p.new_lse_stride_h + t];
  const float mx = fmaxf(la, lb);
  float wa, wb, l;
  if (mx == -INFINITY) {
    wa = wb = 0.f;
    l = -INFINITY;
  } else {
    const float ea = __expf(la - mx), eb = __expf(lb - mx);
    const float inv = 1.f / (ea + eb);
    wa = ea * inv;
    wb = eb * inv;
    l = mx + __logf(ea + eb);
  }
  float* ao = p.acc_o + b * p.acc_stride_b + t * p.acc_stride_t + h * p.acc_stride_h;
  const long long no = b * p.new_stride_b + t * p.new_stride_t + h * p.new_stride_h;
  for (int c = lane * 4; c < p.head_dim; c += 128) {
    float4 x = *reinterpret_cast<const float4*>(ao + c);
    float4 y;
    if constexpr (kKind == 2) {
      y = *reinterpret_cast<const float4*>(static_cast<const float*>(p.new_o) + no + c);
    } else {
      const uint2 r = *reinterpret_cast<const uint2*>(static_cast<const uint16_t*>(p.new_o) + no + c);
      const float2 r0 = unpack2<kKind == 0>(r.x), r1 = unpack2<kKind == 0>(r.y);
      y = make_float4(r0.x, r0.y, r1.x, r1.y);
    }
    // a zero weight must also silence a non-finite value on that side (an untouched accumulator)
    x.x = (wa == 0.f ? 0.f : x.x * wa) + (wb == 0.f ? 0.f : y.x * wb);
    x.y = (wa == 0.f ? 0.f : x.y * wa) + (wb == 0.f ? 0.f : y.y * wb);
    x.z = (wa == 0.f ? 0.f : x.z * wa) + (wb == 0.f ? 0.f : y.z * wb);
    x.w = (wa == 0.f ? 0.f : x.w * wa) + (wb == 0.f ? 0.f : y.w * wb);
    *reinterpret_cast<float4*>(ao + c) = x;
  }
  __syncwarp();
  if (lane == 0) *la_ptr = static_cast<LseT>(l);
}

// acc += recv; 4 elements per thread.  kind: 0 bf16, 1 fp16, 2 float
template <int kKind>
__global__ void halo_acc_kernel(float* __restrict__ acc, long long acc_sb, const void* __restrict__ recv,
                                long long recv_sb, long long vec_per_batch, long long n_vec) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n_vec) return;
  const long long b = i / vec_per_batch, v = i % vec_per_batch;
  float4* a = reinterpret_cast<float4*>(acc + b * acc_sb) + v;
  float4 x = *a;
  if constexpr (kKind == 2) {
    const float4 r = *(reinterpret_cast<const float4*>(static_cast<const float*>(recv) + b * recv_sb) + v);
    x.x += r.x; x.y += r.y; x.z += r.z; x.w += r.w;
  } else {
    const uint2 r = *(reinterpret_cast<const uint2*>(static_cast<const uint16_t*>(recv) + b * recv_sb) + v);
    const float2 r0 = unpack2<kKind == 0>(r.x), r1 = unpack2<kKind == 0>(r.y);
    x.x += r0.x; x.y += r0.y; x.z += r1.x; x.w += r1.y;
  }
  *a = x;
}

// dst = round(acc + recv), nothing written back to acc: the last addition into an accumulator and its
// final rounding in one pass.  kind of recv as above.
template <int kKind, bool kBf16>
__global__ void halo_acc_cast_kernel(uint16_t* __restrict__ dst, long long dst_sb, const float* __restrict__ acc,
                                     long long acc_sb, const void* __restrict__ recv, long long recv_sb,
                                     long long vec_per_batch, long long n_vec) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n_vec) return;
  const long long b = i / vec_per_batch, v = i % vec_per_batch;
  float4 x = *(reinterpret_cast<const float4*>(acc + b * acc_sb) + v);
  if constexpr (kKind == 2) {
    const float4 r = *(reinterpret_cast<const float4*>(static_cast<const float*>(recv) + b * recv_sb) + v);
    x.x += r.x; x.y += r.y; x.z += r.z; x.w += r.w;
  } else {
    const uint2 r = *(reinterpret_cast<const uint2*>(static_cast<const uint16_t*>(recv) + b * recv_sb) + v);
    const float2 r0 = unpack2<kKind == 0>(r.x), r1 = unpack2<kKind == 0>(r.y);
    x.x += r0.x; x.y += r0.y; x.z += r1.x; x.w += r1.y;
  }
  uint2 o;
  o.x = pack2f<kBf16>(x.x, x.y);
  o.y = pack2f<kBf16>(x.z, x.w);
  *(reinterpret_cast<uint2*>(dst + b * dst_sb) + v) = o;
}

template <bool kBf16>
__global__ void cast_kernel(uint16_t* __restrict__ dst, long long dst_sb, const float* __restrict__ src,
                            long long src_sb, long long vec_per_batch, long long n_vec) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n_vec) return;
  const long long b = i / vec_per_batch, v = i % vec_per_batch;
  const float4 x = *(reinterpret_cast<const float4*>(src + b * src_sb) + v);
  uint2 o;
  o.x = pack2f<kBf16>(x.x, x.y);
  o.y = pack2f<kBf16>(x.z, x.w);
  *(reinterpret_cast<uint2*>(dst + b * dst_sb) + v) = o;
}

int check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_error("%s: launch: %s", what, cudaGetErrorString(e));
    return RSWA_E_CUDA;
  }
  return RSWA_OK;
}

}  // namespace

int launch_delta(const rswa_bwd_params_t& p, float* delta, float* lse2, int q_len_pad, cudaStream_t stream) {
  const rswa_geom_t& g = p.g;
  const long long tasks = static_cast<long long>(g.batch) * g.n_q_heads * (q_len_pad / 32);  // one warp each
  const int threads = 256;
  const long long blocks = (tasks * 32 + threads - 1) / threads;
  auto kern = g.dtype == RSWA_DTYPE_BF16 ? delta_kernel<true> : delta_kernel<false>;
  kern<<<static_cast<unsigned>(blocks), threads, 0, stream>>>(
      static_cast<const uint16_t*>(p.out), p.o_stride_b, p.o_stride_t, p.o_stride_h,
      static_cast<const uint16_t*>(p.dout), p.do_stride_b, p.do_stride_t, p.do_stride_h, p.lse, p.lse_stride_b,
      p.lse_stride_h, delta, lse2, g.batch, g.q_len, g.n_q_heads, q_len_pad);
  return check_launch("rswa_bwd(delta)");
}

}  // namespace rswa

using namespace rswa;

extern "C" int rswa_merge(const rswa_merge_params_t* p, void* stream) {
  if (!p || !p->o_a || !p->o_b || !p->o || !p->lse_a || !p->lse_b || !p->lse) {
    set_error("rswa_merge: null argument");
    return RSWA_E_ARG;
  }
  if (p->head_dim != kHeadDim || (p->dtype != RSWA_DTYPE_BF16 && p->dtype != RSWA_DTYPE_FP16)) {
    set_error("rswa_merge: head_dim must be 128 and dtype bf16/fp16");
    return RSWA_E_UNSUPPORTED;
  }
  if (p->batch <= 0 || p->q_len <= 0 || p->n_heads <= 0) {
    set_error("rswa_merge: extents must be positive");
    return RSWA_E_ARG;
  }
  const long long strides[9] = {p->oa_stride_b, p->oa_stride_t, p->oa_stride_h, p->ob_stride_b, p->ob_stride_t,
                                p->ob_stride_h, p->o_stride_b,  p->o_stride_t,  p->o_stride_h};
  for (long long s : strides) {
    if (s % 8) {
      set_error("rswa_merge: strides must be multiples of 8 elements");
      return RSWA_E_ARG;
    }
  }
  if ((reinterpret_cast<uintptr_t>(p->o_a) | reinterpret_cast<uintptr_t>(p->o_b) |
       reinterpret_cast<uintptr_t>(p->o)) & 15) {
    set_error("rswa_merge: pointers must be 16-byte aligned");
    return RSWA_E_ARG;
  }
  const long long n_tasks = static_cast<long long>(p->batch) * p->n_heads * ((p->q_len + 31) / 32);  // one warp each
  const long long n_vec = n_tasks * 32;
  const int threads = 256;
  auto kern = p->dtype == RSWA_DTYPE_BF16 ? merge_kernel<true> : merge_kernel<false>;
  kern<<<static_cast<unsigned>((n_vec + threads - 1) / threads), threads, 0, static_cast<cudaStream_t>(stream)>>>(
      *p, n_tasks);
  return check_launch("rswa_merge");
}

extern "C" int rswa_merge_acc(const rswa_merge_acc_params_t* p, void* stream) {
  if (!p || !p->acc_o || !p->new_o || !p->acc_lse || !p->new_lse) {
    set_error("rswa_merge_acc: null argument");
    return RSWA_E_ARG;
  }
  if (p->new_dtype < 0 || p->new_dtype > RSWA_DTYPE_F32 || (p->lse_f64 != 0 && p->lse_f64 != 1)) {
    set_error("rswa_merge_acc: new_dtype must be bf16/fp16/float and lse_f64 0 or 1");
    return RSWA_E_UNSUPPORTED;
  }
  if (p->batch <= 0 || p->q_len <= 0 || p->n_heads <= 0 || p->head_dim <= 0 || (p->head_dim % 4)) {
    set_error("rswa_merge_acc: extents must be positive and head_dim a multiple of 4");
    return RSWA_E_ARG;
  }
  const long long strides[6] = {p->acc_stride_b, p->acc_stride_t, p->acc_stride_h,
                                p->new_stride_b, p->new_stride_t, p->new_stride_h};
  for (long long s : strides) {
    if (s % 4) {
      set_error("rswa_merge_acc: strides must be multiples of 4 elements");
      return RSWA_E_ARG;
    }
  }
  const uintptr_t new_mask = p->new_dtype == RSWA_DTYPE_F32 ? 15 : 7;
  if ((reinterpret_cast<uintptr_t>(p->acc_o) & 15) || (reinterpret_cast<uintptr_t>(p->new_o) & new_mask)) {
    set_error("rswa_merge_acc: the accumulator must be 16-byte aligned, the incoming output 8- (16-bit) or 16-byte");
    return RSWA_E_ARG;
  }
  const long long n_rows = static_cast<long long>(p->batch) * p->q_len * p->n_heads;
  const int threads = 256;
  const unsigned blocks = static_cast<unsigned>((n_rows * 32 + threads - 1) / threads);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int k = p->new_dtype;
  if (p->lse_f64) {
    if (k == 0) merge_acc_kernel<0, double><<<blocks, threads, 0, s>>>(*p, n_rows);
    else if (k == 1) merge_acc_kernel<1, double><<<blocks, threads, 0, s>>>(*p, n_rows);
    else merge_acc_kernel<2, double><<<blocks, threads, 0, s>>>(*p, n_rows);
  } else {
    if (k == 0) merge_acc_kernel<0, float><<<blocks, threads, 0, s>>>(*p, n_rows);
    else if (k == 1) merge_acc_kernel<1, float><<<blocks, threads, 0, s>>>(*p, n_rows);
    else merge_acc_kernel<2, float><<<blocks, threads, 0, s>>>(*p, n_rows);
  }
  return check_launch("rswa_merge_acc");
}

extern "C" int rswa_halo_accumulate(float* acc, int64_t acc_stride_b, const void* recv, int64_t recv_stride_b,
                                    int32_t recv_dtype, int32_t batch, int64_t elems_per_batch, void* stream) {
  if (!acc || !recv || batch <= 0 || elems_per_batch <= 0 || (elems_per_batch % 4) || (acc_stride_b % 4) ||
      (recv_stride_b % 4) || recv_dtype < 0 || recv_dtype > 2 || (reinterpret_cast<uintptr_t>(acc) & 15) ||
      (reinterpret_cast<uintptr_t>(recv) & 15)) {
    set_error("rswa_halo_accumulate: bad argument (need 16-byte alignment and multiples of 4 elements)");
    return RSWA_E_ARG;
  }
  const long long vpb = elems_per_batch / 4, n_vec = vpb * batch;
  const int threads = 256;
  const unsigned blocks = static_cast<unsigned>((n_vec + threads - 1) / threads);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (recv_dtype == 0) halo_acc_kernel<0><<<blocks, threads, 0, s>>>(acc, acc_stride_b, recv, recv_stride_b, vpb, n_vec);
  else if (recv_dtype == 1) halo_acc_kernel<1><<<blocks, threads, 0, s>>>(acc, acc_stride_b, recv, recv_stride_b, vpb, n_vec);
  else halo_acc_kernel<2><<<blocks, threads, 0, s>>>(acc, acc_stride_b, recv, recv_stride_b, vpb, n_vec);
  return check_launch("rswa_halo_accumulate");
}

extern "C" int rswa_cast_from_f32(void* dst, int64_t dst_stride_b, const float* src, int64_t src_stride_b,
                                  int32_t dtype, int32_t batch, int64_t elems_per_batch, void* stream) {
  if (!dst || !src || batch <= 0 || elems_per_batch <= 0 || (elems_per_batch % 4) || (dst_stride_b % 4) ||
      (src_stride_b % 4) || (dtype != 0 && dtype != 1) || (reinterpret_cast<uintptr_t>(dst) & 7) ||
      (reinterpret_cast<uintptr_t>(src) & 15)) {
    set_error("rswa_cast_from_f32: bad argument");
    return RSWA_E_ARG;
  }
  const long long vpb = elems_per_batch / 4, n_vec = vpb * batch;
  const int threads = 256;
  const unsigned blocks = static_cast<unsigned>((n_vec + threads - 1) / threads);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == 0) cast_kernel<true><<<blocks, threads, 0, s>>>(static_cast<uint16_t*>(dst), dst_stride_b, src, src_stride_b, vpb, n_vec);
  else cast_kernel<false><<<blocks, threads, 0, s>>>(static_cast<uint16_t*>(dst), dst_stride_b, src, src_stride_b, vpb, n_vec);
  return check_launch("rswa_cast_from_f32");
}

extern "C" int rswa_halo_accumulate_cast(void* dst, int64_t dst_stride_b, int32_t dst_dtype, const float* acc,
                                         int64_t acc_stride_b, const void* recv, int64_t recv_stride_b,
                                         int32_t recv_dtype, int32_t batch, int64_t elems_per_batch, void* stream) {
  if (!dst || !acc || !recv || batch <= 0 || elems_per_batch <= 0 || (elems_per_batch % 4) || (acc_stride_b % 4) ||
      (recv_stride_b % 4) || (dst_stride_b % 4) || recv_dtype < 0 || recv_dtype > 2 || (dst_dtype != 0 && dst_dtype != 1) ||
      (reinterpret_cast<uintptr_t>(acc) & 15) || (reinterpret_cast<uintptr_t>(recv) & 15) ||
      (reinterpret_cast<uintptr_t>(dst) & 7)) {
    set_error("rswa_halo_accumulate_cast: bad argument (need 16-byte alignment and multiples of 4 elements)");
    return RSWA_E_ARG;
  }
  const long long vpb = elems_per_batch / 4, n_vec = vpb * batch;
  const int threads = 256;
  const unsigned blocks = static_cast<unsigned>((n_vec + threads - 1) / threads);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  uint16_t* d = static_cast<uint16_t*>(dst);
#define RSWA_LAUNCH_ACC_CAST(K, B) \
  halo_acc_cast_kernel<K, B><<<blocks, threads, 0, s>>>(d, dst_stride_b, acc, acc_stride_b, recv, recv_stride_b, vpb, n_vec)
  if (dst_dtype == 0) {
    if (recv_dtype == 0) RSWA_LAUNCH_ACC_CAST(0, true);
    else if (recv_dtype == 1) RSWA_LAUNCH_ACC_CAST(1, true);
    else RSWA_LAUNCH_ACC_CAST(2, true);
  } else {
    if (recv_dtype == 0) RSWA_LAUNCH_ACC_CAST(0, false);
    else if (recv_dtype == 1) RSWA_LAUNCH_ACC_CAST(1, false);
    else RSWA_LAUNCH_ACC_CAST(2, false);
  }
#undef RSWA_LAUNCH_ACC_CAST
  return check_launch("rswa_halo_accumulate_cast");
}
