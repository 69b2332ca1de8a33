// Forward kernel: banded (sliding-window + sink) softmax attention for one 128-row query tile per
// CTA on the sm_100a tensor cores.
//
//   S = Q K^T      tcgen05.mma, both operands in shared memory (K-major), accumulator in TMEM
//   P = softmax    four warps, one query row per thread, read S from TMEM, write P (16-bit) back
//                  into the same TMEM columns
//   O += P V       tcgen05.mma, A = P from TMEM, B = V from shared memory (MN-major)
//
// Key tiles that no row of the query tile can see are never loaded: the visible keys of a query
// tile are one contiguous run of global positions (plus the sink tokens), intersected with each
// KV span.  Two CTAs share an SM (96 KB of shared memory and 256 TMEM columns each) so that one
// CTA's softmax overlaps the other's MMAs.
//
// The math follows the reference's dense oracle (test/test_local_swa.py:51-93): scores scaled by
// softmax_scale, keys outside [p - W, p] masked to -inf (the sink column forced on,
// test/test_local_slm.py:62-64), fp32 softmax, P rounded to the value dtype before P V.
#include "rswa_common.cuh"
#include "tc05.cuh"

namespace rswa {
using namespace tc05;

namespace {

constexpr int kFwdThreads = 192;  // warp 0: TMA, warp 1: MMA, warps 2-5: softmax
constexpr int kFwdTmemCols = 256; // [0,128) S / P, [128,256) O

struct FwdCtl {
  uint64_t q_full, k_full, v_full, s_ready, pv_done, p_ready;
  uint32_t tmem_base;
  int err;
  int n_entries;
  int n_tiles;
  int ent_span[kMaxEntries];
  int ent_first[kMaxEntries];
  int ent_count[kMaxEntries];
};

constexpr int kFwdSmemBytes = 3 * kTileBytes + 1024 /*alignment slack*/ + 1024 /*FwdCtl*/;
static_assert(sizeof(FwdCtl) <= 1024, "control block too large");

template <bool kBf16>
__global__ void __launch_bounds__(kFwdThreads, 2)
rswa_fwd_kernel(const __grid_constant__ FwdKernelParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = smem + kTileBytes;
  uint8_t* sV = smem + 2 * kTileBytes;
  FwdCtl* ctl = reinterpret_cast<FwdCtl*>(smem + 3 * kTileBytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // work item: query tile fastest, then head, then batch row
  int idx = blockIdx.x;
  const int qt = p.q_tile_begin + idx % p.n_q_tiles;
  idx /= p.n_q_tiles;
  const int h = idx % p.hq;
  const int b = idx / p.hq;
  const int hk = h / (p.hq / p.hkv);

  const int row0 = qt * kTile;
  const int n_valid = min(kTile, p.q_len - row0);
  const int p0 = p.q_pos_start + row0;
  const int p_last = p0 + n_valid - 1;

  if (threadIdx.x == 0) {
    mbar_init(&ctl->q_full, 1);
    mbar_init(&ctl->k_full, 1);
    mbar_init(&ctl->v_full, 1);
    mbar_init(&ctl->s_ready, 1);
    mbar_init(&ctl->pv_done, 1);
    mbar_init(&ctl->p_ready, 128);
    ctl->err = 0;
    mbar_fence_init();
    // Key tiles this query tile needs, per span: the sink tiles that lie below the window
    // tiles, then the window tiles.  Tiles are 128-aligned relative to the span start.
    int s0, e0;
    seq_of(p.cu, p.n_seqs, p0, s0, e0);
    const int min_lo = max(s0, p0 - p.window);
    int ne = 0, nt = 0;
    for (int i = 0; i < p.n_spans; ++i) {
      const int a = p.span_pos[i], bnd = a + p.span_len[i];
      int wfirst = -1, wlast = -1;
      const int wl = max(min_lo, a), wh = min(p_last, bnd - 1);
      if (wl <= wh) {
        wfirst = (wl - a) / kTile;
        wlast = (wh - a) / kTile;
      }
      if (p.n_sink > 0) {
        const int sl = max(s0, a), sh = min(min(s0 + p.n_sink - 1, bnd - 1), p_last);
        if (sl <= sh) {
          const int sf = (sl - a) / kTile;
          int slast = (sh - a) / kTile;
          if (wfirst >= 0) slast = min(slast, wfirst - 1);
          if (sf <= slast) {
            ctl->ent_span[ne] = i;
            ctl->ent_first[ne] = sf;
            ctl->ent_count[ne] = slast - sf + 1;
            nt += slast - sf + 1;
            ++ne;
          }
        }
      }
      if (wfirst >= 0) {
        ctl->ent_span[ne] = i;
        ctl->ent_first[ne] = wfirst;
        ctl->ent_count[ne] = wlast - wfirst + 1;
        nt += wlast - wfirst + 1;
        ++ne;
      }
    }
    ctl->n_entries = ne;
    ctl->n_tiles = nt;
  }
  if (warp == 1) {
    tmem_alloc(&ctl->tmem_base, kFwdTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();

  const uint32_t tmem = ctl->tmem_base;
  const uint32_t tS = tmem;
  const uint32_t tO = tmem + 128;
  volatile int* err = &ctl->err;
  const int n_entries = ctl->n_entries;
  const int n_tiles = ctl->n_tiles;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0 && n_tiles > 0) {
      prefetch_tmap(&p.q_map);
      mbar_expect_tx(&ctl->q_full, kTileBytes);
      tma_load_4d(sQ, &p.q_map, &ctl->q_full, 0, h, row0, b);
      tma_load_4d(sQ + kBoxBytes, &p.q_map, &ctl->q_full, 64, h, row0, b);
      int j = 0;
      bool ok = true;
      for (int e = 0; e < n_entries && ok; ++e) {
        const int sp = ctl->ent_span[e];
        for (int t = 0; t < ctl->ent_count[e] && ok; ++t, ++j) {
          const int tok = (ctl->ent_first[e] + t) * kTile;
          // K buffer is free once S(j-1) has been produced from it
          if (j > 0) ok = mbar_wait(&ctl->s_ready, (j - 1) & 1, err, kErrWaitProducer);
          if (!ok) break;
          mbar_expect_tx(&ctl->k_full, kTileBytes);
          tma_load_4d(sK, &p.k_map[sp], &ctl->k_full, 0, hk, tok, b);
          tma_load_4d(sK + kBoxBytes, &p.k_map[sp], &ctl->k_full, 64, hk, tok, b);
          // V buffer is free once O += P(j-1) V(j-1) has completed
          if (j > 0) ok = mbar_wait(&ctl->pv_done, (j - 1) & 1, err, kErrWaitProducer);
          if (!ok) break;
          mbar_expect_tx(&ctl->v_full, kTileBytes);
          tma_load_4d(sV, &p.v_map[sp], &ctl->v_full, 0, hk, tok, b);
          tma_load_4d(sV + kBoxBytes, &p.v_map[sp], &ctl->v_full, 64, hk, tok, b);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0 && n_tiles > 0) {
      constexpr uint32_t idesc_qk = idesc_f16(128, 128, kBf16 ? 1 : 0, 0, 0);
      constexpr uint32_t idesc_pv = idesc_f16(128, 128, kBf16 ? 1 : 0, 0, 1);
      const uint32_t aQ = smem_u32(sQ), aK = smem_u32(sK), aV = smem_u32(sV);
      bool ok = mbar_wait(&ctl->q_full, 0, err, kErrWaitMma);
      for (int j = 0; j < n_tiles && ok; ++j) {
        // P(j-1) shares TMEM columns with S(j): wait until the previous P V has drained
        if (j > 0) ok = mbar_wait(&ctl->pv_done, (j - 1) & 1, err, kErrWaitMma);
        if (!ok) break;
        ok = mbar_wait(&ctl->k_full, j & 1, err, kErrWaitMma);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const uint32_t off = (k >> 2) * kBoxBytes + (k & 3) * 32;
          mma_ss(tS, smem_desc_sw128(aQ + off, 16, 1024), smem_desc_sw128(aK + off, 16, 1024),
                 idesc_qk, k > 0 ? 1u : 0u);
        }
        mma_commit(&ctl->s_ready);
        ok = mbar_wait(&ctl->v_full, j & 1, err, kErrWaitMma);
        if (!ok) break;
        ok = mbar_wait(&ctl->p_ready, j & 1, err, kErrWaitMma);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          mma_ts(tO, tS + k * 8, smem_desc_sw128(aV + k * 2048, kBoxBytes, 1024), idesc_pv,
                 (j > 0 || k > 0) ? 1u : 0u);
        }
        mma_commit(&ctl->pv_done);
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax + epilogue
    const int quad = warp & 3;              // TMEM lane quadrant this warp may touch
    const int row = quad * 32 + lane;       // query row inside the tile
    const uint32_t lane_off = static_cast<uint32_t>(quad * 32) << 16;
    const bool valid = row < n_valid;
    const int pos = p0 + row;
    int s_p = 0, e_p = 0;
    if (valid) seq_of(p.cu, p.n_seqs, pos, s_p, e_p);
    // visible keys: [lo, hi] plus [s_p, sink_end) (both clipped by t <= pos)
    const int hi = valid ? pos : -1;
    const int lo = valid ? max(s_p, pos - p.window) : 0x7fffffff;
    const int sink_end = valid ? s_p + p.n_sink : -0x7fffffff;
    const float sl2 = p.scale_log2;

    float m_ref = -INFINITY;  // reference maximum, in log2 units (already scaled)
    float l_sum = 0.f;
    bool ok = true;
    int j = 0;
    for (int e = 0; e < n_entries && ok; ++e) {
      const int sp = ctl->ent_span[e];
      const int span_pos = p.span_pos[sp];
      const int span_end = span_pos + p.span_len[sp];
      for (int t = 0; t < ctl->ent_count[e] && ok; ++t, ++j) {
        const int kt0 = span_pos + (ctl->ent_first[e] + t) * kTile;
        ok = mbar_wait(&ctl->s_ready, j & 1, err, kErrWaitSoftmax);
        ok = __all_sync(0xffffffffu, ok);  // keep the warp converged for the TMEM accesses
        if (!ok) break;
        tc_fence_after();
        const bool my_mask = !(kt0 >= lo && kt0 + kTile - 1 <= hi && kt0 + kTile - 1 < span_end);
        const bool masked = __any_sync(0xffffffffu, my_mask);

        // pass 1: row maximum of the raw scores
        float mx = -INFINITY;
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t r[32];
          tmem_ld32(tS + lane_off + c * 32, r);
          tmem_ld_wait();
          if (masked) {
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              const int tk = kt0 + c * 32 + i;
              const bool vis = tk <= hi && tk < span_end && (tk >= lo || (tk >= s_p && tk < sink_end));
              mx = fmaxf(mx, vis ? __uint_as_float(r[i]) : -INFINITY);
            }
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) mx = fmaxf(mx, __uint_as_float(r[i]));
          }
        }
        // Lazy rescale: keep the old reference maximum unless the new one exceeds it by more
        // than 2^8, so that O in TMEM is only touched rarely.
        const float mt = mx * sl2;
        float alpha = 1.f;
        const bool grow = mt > m_ref + 8.f;
        if (grow) {
          alpha = ex2f(m_ref - mt);  // 0 when m_ref is -inf
          m_ref = mt;
        }
        if (j > 0 && __any_sync(0xffffffffu, grow)) {
          l_sum *= alpha;
#pragma unroll 1
          for (int c = 0; c < 4; ++c) {
            uint32_t r[32];
            tmem_ld32(tO + lane_off + c * 32, r);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
            tmem_st32(tO + lane_off + c * 32, r);
          }
          tmem_st_wait();
        }
        const float m_use = (m_ref == -INFINITY) ? 0.f : m_ref;

        // pass 2: P = exp2(S * scale_log2 - m), row sum, write P (16-bit) over S
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t r[32];
          tmem_ld32(tS + lane_off + c * 32, r);
          tmem_ld_wait();
          uint32_t pk[16];
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            float s0 = __uint_as_float(r[i]), s1 = __uint_as_float(r[i + 1]);
            if (masked) {
              const int tk = kt0 + c * 32 + i;
              const bool v0 = tk <= hi && tk < span_end && (tk >= lo || (tk >= s_p && tk < sink_end));
              const bool v1 = tk + 1 <= hi && tk + 1 < span_end &&
                              (tk + 1 >= lo || (tk + 1 >= s_p && tk + 1 < sink_end));
              s0 = v0 ? s0 : -INFINITY;
              s1 = v1 ? s1 : -INFINITY;
            }
            const float e0 = ex2f(fmaf(s0, sl2, -m_use));
            const float e1 = ex2f(fmaf(s1, sl2, -m_use));
            l_sum += e0 + e1;
            pk[i >> 1] = pack2<kBf16>(e0, e1);
          }
          tmem_st16(tS + lane_off + c * 16, pk);
        }
        tmem_st_wait();
        tc_fence_before();
        mbar_arrive(&ctl->p_ready);
      }
    }

    // epilogue: O / l -> out, lse
    if (ok && n_tiles > 0) ok = mbar_wait(&ctl->pv_done, (n_tiles - 1) & 1, err, kErrWaitEpilogue);
    ok = __all_sync(0xffffffffu, ok);
    tc_fence_after();
    const bool has = ok && n_tiles > 0 && l_sum > 0.f;
    const float inv = has ? 1.f / l_sum : 0.f;
    uint16_t* orow = reinterpret_cast<uint16_t*>(p.out) + b * p.o_sb +
                     static_cast<long long>(row0 + row) * p.o_st + h * p.o_sh;
#pragma unroll 1
    for (int c = 0; c < 4; ++c) {
      uint32_t r[32];
      if (n_tiles > 0 && ok) {
        tmem_ld32(tO + lane_off + c * 32, r);
        tmem_ld_wait();
      }
      if (valid) {
        uint4* dst = reinterpret_cast<uint4*>(orow + c * 32);
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          uint4 o;
          if (has) {
            o.x = pack2<kBf16>(__uint_as_float(r[v * 8 + 0]) * inv, __uint_as_float(r[v * 8 + 1]) * inv);
            o.y = pack2<kBf16>(__uint_as_float(r[v * 8 + 2]) * inv, __uint_as_float(r[v * 8 + 3]) * inv);
            o.z = pack2<kBf16>(__uint_as_float(r[v * 8 + 4]) * inv, __uint_as_float(r[v * 8 + 5]) * inv);
            o.w = pack2<kBf16>(__uint_as_float(r[v * 8 + 6]) * inv, __uint_as_float(r[v * 8 + 7]) * inv);
          } else {
            o = make_uint4(0, 0, 0, 0);
          }
          dst[v] = o;
        }
      }
    }
    if (valid) {
      p.lse[b * p.l_sb + h * p.l_sh + row0 + row] =
          has ? (m_ref + log2f(l_sum)) * 0.6931471805599453f : -INFINITY;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, kFwdTmemCols);
  }
  if (threadIdx.x == 0 && ctl->err != 0) atomicCAS(p.status, 0, ctl->err);
}

}  // namespace

int launch_fwd(const FwdKernelParams& kp, int dtype, cudaStream_t stream) {
  const long long n_cta = static_cast<long long>(kp.n_q_tiles) * kp.hq * kp.batch;
  if (n_cta <= 0) return RSWA_OK;
  if (n_cta > 0x7fffffffLL) {
    set_error("rswa_fwd: too many query tiles (%lld)", n_cta);
    return RSWA_E_ARG;
  }
  auto kern = dtype == RSWA_DTYPE_BF16 ? rswa_fwd_kernel<true> : rswa_fwd_kernel<false>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kFwdSmemBytes);
  if (e != cudaSuccess) {
    set_error("rswa_fwd: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    return RSWA_E_CUDA;
  }
  kern<<<static_cast<unsigned>(n_cta), kFwdThreads, kFwdSmemBytes, stream>>>(kp);
  e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_error("rswa_fwd: launch: %s", cudaGetErrorString(e));
    return RSWA_E_CUDA;
  }
  return RSWA_OK;
}

}  // namespace rswa
