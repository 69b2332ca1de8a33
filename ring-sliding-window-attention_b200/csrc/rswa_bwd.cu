// Backward kernel: one CTA owns a 128-key tile of one KV head and walks every query tile (and
// every query head of the group) that can see it.  All five products run on the sm_100a tensor
// cores with TMEM accumulators, in the transposed (key-major) form so that P and dS can be fed
// back as the A operand straight from tensor memory:
//
//   S^T  = K Q^T          A = K   (smem, K-major)     B = Q   (smem, K-major)
//   dP^T = V dO^T         A = V   (smem, K-major)     B = dO  (smem, K-major)
//   P^T  = exp2(S^T * scale_log2 - lse),   dS^T = P^T * (dP^T - delta)      (8 warps)
//   dV  += P^T dO         A = P^T (TMEM)              B = dO  (smem, MN-major)
//   dK  += dS^T Q         A = dS^T(TMEM)              B = Q   (smem, MN-major)
//   dQ   = dS K           A = dS^T(smem, MN-major)    B = K   (smem, MN-major)
//
// dK and dV stay in TMEM for the whole CTA (summed over the query heads of the group) and are
// written once; dQ tiles are added into an fp32 accumulator in global memory with vector
// reductions and converted afterwards.  P is recomputed from the saved log-sum-exp, and delta is
// rowsum(dO * O), which is what makes a per-span backward against the FINAL out/lse exact
// (the property the reference's per-hop backward relies on, ring_swa/ops/attn.py:63-126).
//
// TMEM columns: [0,128) dK, [128,256) dV, [256,384) S^T then P^T | dS^T, [384,512) dP^T then dQ.
#include "rswa_common.cuh"
#include "tc05.cuh"

namespace rswa {
using namespace tc05;

namespace {

constexpr int kBwdThreads = 320;  // warp 0: TMA, warp 1: MMA, warps 2-9: compute
constexpr int kBwdTmemCols = 512;

struct BwdCtl {
  uint64_t kv_full, qdo_full[2], stage_free[2], sdp_ready, pds_ready, mma2_done, dq_done;
  uint32_t tmem_base;
  int err;
  int qt_first, n_qt;
};

// K, V, 2 x (Q, dO), dS  +  2 x (lse, delta) rows  +  control
constexpr int kBwdSmemTiles = 7 * kTileBytes;
constexpr int kBwdSmemBytes = kBwdSmemTiles + 2 * 2 * kTile * 4 + 256;
static_assert(sizeof(BwdCtl) <= 256, "control block too large");
static_assert(kBwdSmemBytes <= 232448, "shared memory budget");

__device__ __forceinline__ void red_add_v4(float* addr, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d)
               : "memory");
}
__device__ __forceinline__ void bar_sync_compute() { asm volatile("bar.sync 1, 256;" ::: "memory"); }
__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

template <bool kBf16>
__global__ void __launch_bounds__(kBwdThreads, 1)
rswa_bwd_kernel(const __grid_constant__ BwdKernelParams p, int total_tiles) {
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* sK = smem;
  uint8_t* sV = smem + kTileBytes;
  uint8_t* sQ = smem + 2 * kTileBytes;   // two stages
  uint8_t* sDO = smem + 4 * kTileBytes;  // two stages
  uint8_t* sDS = smem + 6 * kTileBytes;
  float* sLse = reinterpret_cast<float*>(smem + kBwdSmemTiles);  // [2][128]
  float* sDelta = sLse + 2 * kTile;                              // [2][128]
  BwdCtl* ctl = reinterpret_cast<BwdCtl*>(smem + kBwdSmemTiles + 2 * 2 * kTile * 4);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // work item: batch row fastest, then KV head, then key tile (tiles of the first span first)
  int idx = blockIdx.x;
  const int b = idx % p.batch;
  idx /= p.batch;
  const int hk = idx % p.hkv;
  const int kt_g = idx / p.hkv;
  int sp = 0;
  while (sp + 1 < p.n_spans && kt_g >= p.span_tile0[sp + 1]) ++sp;
  const int kt = kt_g - p.span_tile0[sp];
  const int key0 = kt * kTile;  // token offset inside the span
  const int n_valid_k = min(kTile, p.span_len[sp] - key0);
  const int t0 = p.span_pos[sp] + key0;
  const int group = p.hq / p.hkv;
  const int q_end_pos = p.q_pos_start + p.q_len;  // exclusive

  if (threadIdx.x == 0) {
    mbar_init(&ctl->kv_full, 1);
    mbar_init(&ctl->qdo_full[0], 1);
    mbar_init(&ctl->qdo_full[1], 1);
    mbar_init(&ctl->stage_free[0], 1);
    mbar_init(&ctl->stage_free[1], 1);
    mbar_init(&ctl->sdp_ready, 1);
    mbar_init(&ctl->pds_ready, 256);
    mbar_init(&ctl->mma2_done, 1);
    mbar_init(&ctl->dq_done, 256);
    ctl->err = (smem_u32(smem) & 1023u) ? 199 : 0;
    mbar_fence_init();
    // query tiles that can see at least one key of this tile
    const int t_last = t0 + n_valid_k - 1;
    int s_last, e_last;
    seq_of(p.cu, p.n_seqs, t_last, s_last, e_last);
    int pmax;
    if (p.n_sink > 0 && s_last + p.n_sink > t0) {
      pmax = e_last - 1;  // the tile holds a sink token: every later query of that sequence
    } else {
      pmax = (e_last - 1 - t_last > p.window) ? t_last + p.window : e_last - 1;
    }
    const int q_lo = max(t0, p.q_pos_start);
    const int q_hi = min(pmax, q_end_pos - 1);
    if (q_lo <= q_hi) {
      ctl->qt_first = (q_lo - p.q_pos_start) / kTile;
      ctl->n_qt = (q_hi - p.q_pos_start) / kTile - ctl->qt_first + 1;
    } else {
      ctl->qt_first = 0;
      ctl->n_qt = 0;
    }
  }
  if (warp == 1) {
    tmem_alloc(&ctl->tmem_base, kBwdTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();

  const uint32_t tmem = ctl->tmem_base;
  const uint32_t tDK = tmem, tDV = tmem + 128, tA = tmem + 256, tB = tmem + 384;
  const uint32_t tP = tA, tDS = tA + 64;
  volatile int* err = &ctl->err;
  const int qt_first = ctl->qt_first;
  const int n_qt = (ctl->err != 0) ? 0 : ctl->n_qt;
  const int n_iter = n_qt * group;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0 && n_iter > 0) {
      mbar_expect_tx(&ctl->kv_full, 2 * kTileBytes);
      tma_load_4d(sK, &p.k_map[sp], &ctl->kv_full, 0, hk, key0, b);
      tma_load_4d(sK + kBoxBytes, &p.k_map[sp], &ctl->kv_full, 64, hk, key0, b);
      tma_load_4d(sV, &p.v_map[sp], &ctl->kv_full, 0, hk, key0, b);
      tma_load_4d(sV + kBoxBytes, &p.v_map[sp], &ctl->kv_full, 64, hk, key0, b);
      bool ok = true;
      for (int it = 0; it < n_iter && ok; ++it) {
        const int st = it & 1;
        const int h = hk * group + it / n_qt;
        const int row0 = (qt_first + it % n_qt) * kTile;
        if (it >= 2) ok = mbar_wait(&ctl->stage_free[st], ((it >> 1) - 1) & 1, err, kErrWaitProducer);
        if (!ok) break;
        mbar_expect_tx(&ctl->qdo_full[st], 2 * kTileBytes);
        uint8_t* q_dst = sQ + st * kTileBytes;
        uint8_t* do_dst = sDO + st * kTileBytes;
        tma_load_4d(q_dst, &p.q_map, &ctl->qdo_full[st], 0, h, row0, b);
        tma_load_4d(q_dst + kBoxBytes, &p.q_map, &ctl->qdo_full[st], 64, h, row0, b);
        tma_load_4d(do_dst, &p.do_map, &ctl->qdo_full[st], 0, h, row0, b);
        tma_load_4d(do_dst + kBoxBytes, &p.do_map, &ctl->qdo_full[st], 64, h, row0, b);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0 && n_iter > 0) {
      constexpr int bf = kBf16 ? 1 : 0;
      constexpr uint32_t id_kk = idesc_f16(128, 128, bf, 0, 0);  // both operands K-major
      constexpr uint32_t id_tn = idesc_f16(128, 128, bf, 0, 1);  // A from TMEM, B MN-major
      constexpr uint32_t id_nn = idesc_f16(128, 128, bf, 1, 1);  // both MN-major
      const uint32_t aK = smem_u32(sK), aV = smem_u32(sV), aDS = smem_u32(sDS);
      bool ok = mbar_wait(&ctl->kv_full, 0, err, kErrWaitMma);
      for (int it = 0; it < n_iter && ok; ++it) {
        const int st = it & 1;
        const uint32_t aQ = smem_u32(sQ + st * kTileBytes), aDO = smem_u32(sDO + st * kTileBytes);
        ok = mbar_wait(&ctl->qdo_full[st], (it >> 1) & 1, err, kErrWaitMma);
        if (!ok) break;
        // P^T / dS^T of the previous iteration live where S^T goes: wait for the MMAs reading them
        if (it > 0) ok = mbar_wait(&ctl->mma2_done, (it - 1) & 1, err, kErrWaitMma);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const uint32_t off = (k >> 2) * kBoxBytes + (k & 3) * 32;
          mma_ss(tA, smem_desc_sw128(aK + off, 16, 1024), smem_desc_sw128(aQ + off, 16, 1024), id_kk,
                 k > 0 ? 1u : 0u);
        }
        // dQ of the previous iteration lives where dP^T goes: wait until it has been read out
        if (it > 0) ok = mbar_wait(&ctl->dq_done, (it - 1) & 1, err, kErrWaitMma);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const uint32_t off = (k >> 2) * kBoxBytes + (k & 3) * 32;
          mma_ss(tB, smem_desc_sw128(aV + off, 16, 1024), smem_desc_sw128(aDO + off, 16, 1024), id_kk,
                 k > 0 ? 1u : 0u);
        }
        mma_commit(&ctl->sdp_ready);
        ok = mbar_wait(&ctl->pds_ready, it & 1, err, kErrWaitMma);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < 8; ++k) {  // dV += P^T dO
          mma_ts(tDV, tP + k * 8, smem_desc_sw128(aDO + k * 2048, kBoxBytes, 1024), id_tn,
                 (it > 0 || k > 0) ? 1u : 0u);
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) {  // dK += dS^T Q
          mma_ts(tDK, tDS + k * 8, smem_desc_sw128(aQ + k * 2048, kBoxBytes, 1024), id_tn,
                 (it > 0 || k > 0) ? 1u : 0u);
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) {  // dQ = dS K
          mma_ss(tB, smem_desc_sw128(aDS + k * 2048, kBoxBytes, 1024),
                 smem_desc_sw128(aK + k * 2048, kBoxBytes, 1024), id_nn, k > 0 ? 1u : 0u);
        }
        mma_commit(&ctl->mma2_done);
        mma_commit(&ctl->stage_free[st]);
      }
    }
  } else {
    // ------------------------------------------------------------------ compute warps
    const int quad = warp & 3;
    const int half = (warp - 2) >> 2;            // which 64 columns of the 128 this warp handles
    const int row = quad * 32 + lane;            // key row (S^T, dK, dV) or query row (dQ)
    const int ctid = threadIdx.x - 64;           // 0..255
    const uint32_t lane_off = static_cast<uint32_t>(quad * 32) << 16;
    const bool valid_k = row < n_valid_k;
    const int t = valid_k ? t0 + row : 0x7fffffff;
    int p_hi = -1;
    if (valid_k) {
      int s_t, e_t;
      seq_of(p.cu, p.n_seqs, t, s_t, e_t);
      const bool is_sink = t < s_t + p.n_sink;
      p_hi = (is_sink || e_t - 1 - t <= p.window) ? e_t - 1 : t + p.window;
      p_hi = min(p_hi, q_end_pos - 1);
    }
    const float sl2 = p.scale_log2;
    const uint32_t ds_row = smem_u32(sDS) + half * kBoxBytes + row * 128;
    bool ok = true;

    for (int it = 0; it < n_iter && ok; ++it) {
      const int h = hk * group + it / n_qt;
      const int qrow0 = (qt_first + it % n_qt) * kTile;
      const int pq0 = p.q_pos_start + qrow0;
      float* lse_s = sLse + (it & 1) * kTile;
      float* del_s = sDelta + (it & 1) * kTile;
      {
        const int qi = ctid & 127;
        const bool qv = qrow0 + qi < p.q_len;
        if (ctid < 128) {
          lse_s[qi] = qv ? p.lse[b * p.l_sb + h * p.l_sh + qrow0 + qi] * 1.4426950408889634f : INFINITY;
        } else {
          del_s[qi] = qv ? p.delta[b * p.d_sb + h * p.d_sh + qrow0 + qi] : 0.f;
        }
      }
      ok = mbar_wait(&ctl->sdp_ready, it & 1, err, kErrWaitSoftmax);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      uint32_t s[64], dp[64];
      {
        uint32_t(&s0)[32] = *reinterpret_cast<uint32_t(*)[32]>(&s[0]);
        uint32_t(&s1)[32] = *reinterpret_cast<uint32_t(*)[32]>(&s[32]);
        uint32_t(&d0)[32] = *reinterpret_cast<uint32_t(*)[32]>(&dp[0]);
        uint32_t(&d1)[32] = *reinterpret_cast<uint32_t(*)[32]>(&dp[32]);
        tmem_ld32(tA + lane_off + half * 64, s0);
        tmem_ld32(tA + lane_off + half * 64 + 32, s1);
        tmem_ld32(tB + lane_off + half * 64, d0);
        tmem_ld32(tB + lane_off + half * 64 + 32, d1);
        tmem_ld_wait();
      }
      tc_fence_before();
      bar_sync_compute();  // lse/delta rows are in smem; every warp has read S^T and dP^T
      tc_fence_after();

      const bool full = (pq0 >= t) && (pq0 + kTile - 1 <= p_hi);
      const bool masked = !__all_sync(0xffffffffu, full);
      uint32_t ppk[32], dpk[32];
#pragma unroll
      for (int i = 0; i < 64; i += 2) {
        const int q = half * 64 + i;
        const float2 l2 = *reinterpret_cast<const float2*>(lse_s + q);
        const float2 dl = *reinterpret_cast<const float2*>(del_s + q);
        float p0 = ex2f(fmaf(__uint_as_float(s[i]), sl2, -l2.x));
        float p1 = ex2f(fmaf(__uint_as_float(s[i + 1]), sl2, -l2.y));
        if (masked) {
          const int pq = pq0 + q;
          p0 = (pq >= t && pq <= p_hi) ? p0 : 0.f;
          p1 = (pq + 1 >= t && pq + 1 <= p_hi) ? p1 : 0.f;
        }
        const float ds0 = p0 * (__uint_as_float(dp[i]) - dl.x);
        const float ds1 = p1 * (__uint_as_float(dp[i + 1]) - dl.y);
        ppk[i >> 1] = pack2<kBf16>(p0, p1);
        dpk[i >> 1] = pack2<kBf16>(ds0, ds1);
      }
      tmem_st32(tP + lane_off + half * 32, ppk);
      tmem_st32(tDS + lane_off + half * 32, dpk);
      // dS^T also goes to shared memory ([key][query], query contiguous, 128-byte swizzle) as the
      // A operand of dQ = dS K
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        st_shared_v4(ds_row + ((c ^ (row & 7)) << 4), dpk[c * 4], dpk[c * 4 + 1], dpk[c * 4 + 2],
                     dpk[c * 4 + 3]);
      }
      tmem_st_wait();
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(&ctl->pds_ready);

      // dQ tile -> fp32 accumulator in global memory
      ok = mbar_wait(&ctl->mma2_done, it & 1, err, kErrWaitEpilogue);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      {
        const bool qv = qrow0 + row < p.q_len;
        float* dst = p.dq_acc + ((static_cast<long long>(b) * p.q_len + qrow0 + row) * p.hq + h) * kHeadDim +
                     half * 64;
#pragma unroll 1
        for (int c = 0; c < 2; ++c) {
          uint32_t r[32];
          tmem_ld32(tB + lane_off + half * 64 + c * 32, r);
          tmem_ld_wait();
          if (qv) {
#pragma unroll
            for (int v = 0; v < 8; ++v) {
              red_add_v4(dst + c * 32 + v * 4, __uint_as_float(r[v * 4]), __uint_as_float(r[v * 4 + 1]),
                         __uint_as_float(r[v * 4 + 2]), __uint_as_float(r[v * 4 + 3]));
            }
          }
        }
      }
      tc_fence_before();
      mbar_arrive(&ctl->dq_done);
    }

    // epilogue: dK (scaled) and dV for this key tile
    ok = __all_sync(0xffffffffu, ok);
    if (ok && ctl->err == 0) {
      const long long off = b * p.dkv_sb[sp] + static_cast<long long>(key0 + row) * p.dkv_st[sp] +
                            hk * p.dkv_sh[sp] + half * 64;
#pragma unroll 1
      for (int which = 0; which < 2; ++which) {
        const uint32_t tsrc = which == 0 ? tDK : tDV;
        const float mul = which == 0 ? p.scale : 1.f;
        void* base = which == 0 ? p.dk[sp] : p.dv[sp];
#pragma unroll 1
        for (int c = 0; c < 2; ++c) {
          uint32_t r[32];
          if (n_iter > 0) {
            tmem_ld32(tsrc + lane_off + half * 64 + c * 32, r);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = 0u;
          }
          if (valid_k) {
            if (p.grad_fp32[sp]) {
              float4* dst = reinterpret_cast<float4*>(static_cast<float*>(base) + off + c * 32);
#pragma unroll
              for (int v = 0; v < 8; ++v) {
                dst[v] = make_float4(__uint_as_float(r[v * 4]) * mul, __uint_as_float(r[v * 4 + 1]) * mul,
                                     __uint_as_float(r[v * 4 + 2]) * mul, __uint_as_float(r[v * 4 + 3]) * mul);
              }
            } else {
              uint4* dst = reinterpret_cast<uint4*>(static_cast<uint16_t*>(base) + off + c * 32);
#pragma unroll
              for (int v = 0; v < 4; ++v) {
                uint4 o;
                o.x = pack2<kBf16>(__uint_as_float(r[v * 8 + 0]) * mul, __uint_as_float(r[v * 8 + 1]) * mul);
                o.y = pack2<kBf16>(__uint_as_float(r[v * 8 + 2]) * mul, __uint_as_float(r[v * 8 + 3]) * mul);
                o.z = pack2<kBf16>(__uint_as_float(r[v * 8 + 4]) * mul, __uint_as_float(r[v * 8 + 5]) * mul);
                o.w = pack2<kBf16>(__uint_as_float(r[v * 8 + 6]) * mul, __uint_as_float(r[v * 8 + 7]) * mul);
                dst[v] = o;
              }
            }
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, kBwdTmemCols);
  }
  if (threadIdx.x == 0 && ctl->err != 0) atomicCAS(p.status, 0, ctl->err);
}

}  // namespace

int launch_bwd(const BwdKernelParams& kp, int dtype, int total_key_tiles, cudaStream_t stream) {
  const long long n_cta = static_cast<long long>(total_key_tiles) * kp.hkv * kp.batch;
  if (n_cta <= 0) return RSWA_OK;
  if (n_cta > 0x7fffffffLL) {
    set_error("rswa_bwd: too many key tiles (%lld)", n_cta);
    return RSWA_E_ARG;
  }
  auto kern = dtype == RSWA_DTYPE_BF16 ? rswa_bwd_kernel<true> : rswa_bwd_kernel<false>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kBwdSmemBytes);
  if (e != cudaSuccess) {
    set_error("rswa_bwd: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    return RSWA_E_CUDA;
  }
  kern<<<static_cast<unsigned>(n_cta), kBwdThreads, kBwdSmemBytes, stream>>>(kp, total_key_tiles);
  e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_error("rswa_bwd: launch: %s", cudaGetErrorString(e));
    return RSWA_E_CUDA;
  }
  return RSWA_OK;
}

}  // namespace rswa
