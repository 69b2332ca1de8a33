// dQ kernel: the query-stationary half of the backward pass.
//
// One CTA owns one 128-row query tile of one head and walks the key tiles its rows can see, over
// every KV span of the call (sink | halo | local), so that dQ is accumulated on chip and written
// exactly once -- no atomics, no fp32 accumulator in global memory:
//
//   S  = Q K^T          A = Q  (smem, K-major)   B = K (smem, K-major)     two TMEM buffers
//   dP = dO V^T         A = dO (smem, K-major)   B = V (smem, K-major)
//   P  = exp2(S * scale_log2 - lse2[row]),  dS = P * (dP - delta[row])      (8 compute warps)
//   dQ += dS K          A = dS (TMEM, written over S)   B = K (smem, MN-major)
//
// P is recomputed from the final log-sum-exp, so the result is exact for any set of spans
// (the property the reference's per-hop backward relies on, ring_swa/ops/attn.py:63-126).
// S of the next key tile is produced while the compute warps still work on the current one (two S
// buffers), dP of the next tile as soon as the current dP has been read.  Two warps issue MMAs
// (S and dQ from one, dP from the other) because the issue path, not the tensor pipe, is what a
// single thread saturates first.
// TMEM: [0,128) S_0/dS_0, [128,256) S_1/dS_1, [256,384) dP, [384,512) dQ.
#include "rswa_common.cuh"
#include "rswa_tiles.cuh"
#include "tc05.cuh"

namespace rswa {
using namespace tc05;

namespace {

constexpr int kDqThreads = 384;  // warp 0 TMA, warps 1-2 MMA, warp 3 idle, warps 4-11 compute
constexpr int kDqTmemCols = 512;
constexpr int kDqKStages = 3;
constexpr int kDqSmemTiles = 7 * kTileBytes;  // Q, dO, K x 3, V x 2
constexpr int kDqCompute = 256;

struct DqCtl {
  uint64_t q_full, k_full[kDqKStages], v_full[2], k_free[kDqKStages], v_free[2];
  uint64_t s_ready[2], dp_ready, dp_loaded, ds_ready, done;
  uint32_t tmem_base;
  int err;
  QBlockGeom geom;
};

constexpr int kDqSmemBytes = kDqSmemTiles + 1024;
static_assert(sizeof(DqCtl) <= 1024, "control block too large");
static_assert(kDqSmemBytes <= 232448, "shared memory budget");

__device__ __forceinline__ void bar_sync_pair(int id) { asm volatile("bar.sync %0, 64;" ::"r"(id) : "memory"); }

template <bool kBf16>
__global__ void __launch_bounds__(kDqThreads, 1)
rswa_dq_kernel(const __grid_constant__ BwdKernelParams p, int n_q_tiles) {
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* sQ = smem;
  uint8_t* sDO = smem + kTileBytes;
  uint8_t* sK = smem + 2 * kTileBytes;  // three stages
  uint8_t* sV = smem + 5 * kTileBytes;  // two stages
  DqCtl* ctl = reinterpret_cast<DqCtl*>(smem + kDqSmemTiles);
  QBlockGeom* geom = &ctl->geom;

  // a device-side error was already reported on this stream: do not pile further time-outs on it
  if (__syncthreads_or(*reinterpret_cast<volatile int*>(p.status) != 0)) return;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // work item: query tile fastest, then head, then batch row
  int idx = blockIdx.x;
  const int qt = idx % n_q_tiles;
  idx /= n_q_tiles;
  const int h = idx % p.hq;
  const int b = idx / p.hq;
  const int hk = h / (p.hq / p.hkv);
  const int row0 = qt * kTile;

  if (threadIdx.x == 0) {
    mbar_init(&ctl->q_full, 1);
    for (int i = 0; i < kDqKStages; ++i) {
      mbar_init(&ctl->k_full[i], 1);
      mbar_init(&ctl->k_free[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&ctl->v_full[i], 1);
      mbar_init(&ctl->v_free[i], 1);
      mbar_init(&ctl->s_ready[i], 1);
    }
    mbar_init(&ctl->dp_ready, 1);
    mbar_init(&ctl->dp_loaded, kDqCompute);
    mbar_init(&ctl->ds_ready, kDqCompute);
    mbar_init(&ctl->done, 1);
    ctl->err = (smem_u32(smem) & 1023u) ? 199 : 0;
    mbar_fence_init();
    // a block of one query tile: the second tile of the geometry stays empty
    qblock_geometry<kTile>(geom, p.cu, p.n_seqs, p.n_spans, p.span_pos, p.span_len, p.q_pos_start, p.q_len,
                           p.window, p.n_sink, qt, qt + 1);
  }
  if (warp == 1) {
    tmem_alloc(&ctl->tmem_base, kDqTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();

  const uint32_t tmem = ctl->tmem_base;
  const uint32_t tDP = tmem + 256, tDQ = tmem + 384;
  volatile int* err = &ctl->err;
  const int n_tiles = (ctl->err != 0) ? 0 : geom->n_tiles;

  if (warp < 4) {
    setmaxnreg_dec<64>();
    if (warp == 0 && lane == 0 && n_tiles > 0) {
      // ------------------------------------------------------------------ TMA producer
      mbar_expect_tx(&ctl->q_full, 2 * kTileBytes);
      tma_load_4d(sQ, &p.q_map, &ctl->q_full, 0, h, row0, b);
      tma_load_4d(sQ + kBoxBytes, &p.q_map, &ctl->q_full, 64, h, row0, b);
      tma_load_4d(sDO, &p.do_map, &ctl->q_full, 0, h, row0, b);
      tma_load_4d(sDO + kBoxBytes, &p.do_map, &ctl->q_full, 64, h, row0, b);
      TileCursor c;
      cursor_begin<kTile>(geom, p.span_pos, p.span_len, c);
      bool ok = true;
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int sk = j % kDqKStages, sv = j & 1;
        if (j >= kDqKStages) ok = mbar_wait<200>(&ctl->k_free[sk], ((j / kDqKStages) - 1) & 1, err, kErrWaitProducer);
        if (!ok) break;
        mbar_expect_tx(&ctl->k_full[sk], kTileBytes);
        tma_load_4d(sK + sk * kTileBytes, &p.k_map[c.span], &ctl->k_full[sk], 0, hk, c.tok, b);
        tma_load_4d(sK + sk * kTileBytes + kBoxBytes, &p.k_map[c.span], &ctl->k_full[sk], 64, hk, c.tok, b);
        if (j >= 2) ok = mbar_wait<200>(&ctl->v_free[sv], ((j >> 1) - 1) & 1, err, kErrWaitProducer);
        if (!ok) break;
        mbar_expect_tx(&ctl->v_full[sv], kTileBytes);
        tma_load_4d(sV + sv * kTileBytes, &p.v_map[c.span], &ctl->v_full[sv], 0, hk, c.tok, b);
        tma_load_4d(sV + sv * kTileBytes + kBoxBytes, &p.v_map[c.span], &ctl->v_full[sv], 64, hk, c.tok, b);
        cursor_next<kTile>(geom, p.span_pos, p.span_len, c, j + 1 < n_tiles);
      }
    } else if (warp == 1 && lane == 0 && n_tiles > 0) {
      // ------------------------------------------------------------------ MMA issuer 1: S and dQ
      constexpr uint32_t id_kk = idesc_f16(128, 128, kBf16 ? 1 : 0, 0, 0);
      constexpr uint32_t id_tn = idesc_f16(128, 128, kBf16 ? 1 : 0, 0, 1);
      constexpr uint32_t kTile16 = kTileBytes >> 4;
      const uint64_t dQd = smem_desc_sw128(smem_u32(sQ), 16, 1024);
      const uint64_t dKk = smem_desc_sw128(smem_u32(sK), 16, 1024);        // K as K-major B of S
      const uint64_t dKm = smem_desc_sw128(smem_u32(sK), kBoxBytes, 1024); // K as MN-major B of dQ
      bool ok = mbar_wait<40>(&ctl->q_full, 0, err, kErrWaitMma);
      if (ok) ok = mbar_wait<40>(&ctl->k_full[0], 0, err, kErrWaitMma);
      if (ok) {
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const uint32_t off = ((k >> 2) * kBoxBytes + (k & 3) * 32) >> 4;
          mma_ss(tmem, dQd + off, dKk + off, id_kk, k > 0 ? 1u : 0u);
        }
        mma_commit(&ctl->s_ready[0]);
      }
      for (int j = 0; j < n_tiles && ok; ++j) {
        const bool more = j + 1 < n_tiles;
        if (more) {
          // S of the next tile into the other buffer; its previous content (dS of tile j-1) was
          // consumed by a product this thread issued earlier
          const int sk = (j + 1) % kDqKStages;
          ok = mbar_wait<40>(&ctl->k_full[sk], ((j + 1) / kDqKStages) & 1, err, kErrWaitMma);
          if (!ok) break;
          tc_fence_after();
          const uint64_t dKs = dKk + sk * kTile16;
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const uint32_t off = ((k >> 2) * kBoxBytes + (k & 3) * 32) >> 4;
            mma_ss(tmem + 128 * ((j + 1) & 1), dQd + off, dKs + off, id_kk, k > 0 ? 1u : 0u);
          }
          mma_commit(&ctl->s_ready[(j + 1) & 1]);
        }
        ok = mbar_wait<40>(&ctl->ds_ready, j & 1, err, kErrWaitMma);
        if (!ok) break;
        tc_fence_after();
        const uint64_t dKj = dKm + (j % kDqKStages) * kTile16;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          mma_ts(tDQ, tmem + 128 * (j & 1) + k * 8, dKj + k * 128, id_tn, (j > 0 || k > 0) ? 1u : 0u);
        }
        mma_commit(&ctl->k_free[j % kDqKStages]);
      }
      if (ok) mma_commit(&ctl->done);
    } else if (warp == 2 && lane == 0 && n_tiles > 0) {
      // ------------------------------------------------------------------ MMA issuer 2: dP
      constexpr uint32_t id_kk = idesc_f16(128, 128, kBf16 ? 1 : 0, 0, 0);
      constexpr uint32_t kTile16 = kTileBytes >> 4;
      const uint64_t dDO = smem_desc_sw128(smem_u32(sDO), 16, 1024);
      const uint64_t dVk = smem_desc_sw128(smem_u32(sV), 16, 1024);
      bool ok = mbar_wait<40>(&ctl->q_full, 0, err, kErrWaitMma);
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int sv = j & 1;
        ok = mbar_wait<40>(&ctl->v_full[sv], (j >> 1) & 1, err, kErrWaitMma);
        // the compute warps must have read dP of the previous tile out of TMEM
        if (ok && j > 0) ok = mbar_wait<40>(&ctl->dp_loaded, (j - 1) & 1, err, kErrWaitMma);
        if (!ok) break;
        tc_fence_after();
        const uint64_t dVs = dVk + sv * kTile16;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const uint32_t off = ((k >> 2) * kBoxBytes + (k & 3) * 32) >> 4;
          mma_ss(tDP, dDO + off, dVs + off, id_kk, k > 0 ? 1u : 0u);
        }
        mma_commit(&ctl->dp_ready);
        mma_commit(&ctl->v_free[sv]);
      }
    }
  } else {
    // -------------------------------------------------------------------- compute warps
    setmaxnreg_inc<216>();  // 128 x 64 + 256 x 216 <= 384 x 168 (the launch allocation)
    const int quad = warp & 3;
    const int half = (warp - 4) >> 2;       // which 64 key columns of the tile this warp handles
    const int row = quad * 32 + lane;       // query row inside the tile
    const uint32_t lane_off = static_cast<uint32_t>(quad * 32) << 16;
    const bool valid = row < geom->n_valid[0];
    const int pos = geom->p0[0] + row;
    int s_p = 0, e_p = 0;
    if (valid) seq_of(p.cu, p.n_seqs, pos, s_p, e_p);
    const int hi = valid ? pos : -1;
    const int lo = valid ? max(s_p, pos - p.window) : 0x7fffffff;
    const int sink_end = valid ? s_p + p.n_sink : -0x7fffffff;
    const long long roff = b * p.d_sb + h * p.d_sh + row0 + row;  // rows are padded to whole tiles
    const float lse2_r = p.lse2[roff];                            // +inf past q_len: P vanishes
    const float delta_r = p.delta[roff];
    const float sl2 = p.scale_log2;
    bool ok = true;
    TileCursor cur;
    cursor_begin<kTile>(geom, p.span_pos, p.span_len, cur);
    for (int j = 0; j < n_tiles && ok; ++j) {
      const int kt0 = cur.kt0 + half * 64;
      const int span_end = cur.kt_last + 1;
      const uint32_t tSj = tmem + 128 * (j & 1) + lane_off;
      ok = mbar_wait(&ctl->s_ready[j & 1], (j >> 1) & 1, err, kErrWaitSoftmax);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      float pr[64];
      {
        uint32_t s0[32], s1[32];
        tmem_ld32(tSj + half * 64, s0);
        tmem_ld32(tSj + half * 64 + 32, s1);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          pr[i] = ex2f(fmaf(__uint_as_float(s0[i]), sl2, -lse2_r));
          pr[i + 32] = ex2f(fmaf(__uint_as_float(s1[i]), sl2, -lse2_r));
        }
      }
      const bool my_mask = !(kt0 >= lo && kt0 + 63 <= hi && kt0 + 63 < span_end);
      if (__any_sync(0xffffffffu, my_mask)) {
#pragma unroll
        for (int i = 0; i < 64; ++i) {
          const int t = kt0 + i;
          const bool vis = t <= hi && t < span_end && (t >= lo || (t >= s_p && t < sink_end));
          pr[i] = vis ? pr[i] : 0.f;
        }
      }
      ok = mbar_wait(&ctl->dp_ready, j & 1, err, kErrWaitSoftmax);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      uint32_t dpk[32];
      {
        uint32_t d0[32], d1[32];
        tmem_ld32(tDP + lane_off + half * 64, d0);
        tmem_ld32(tDP + lane_off + half * 64 + 32, d1);
        tmem_ld_wait();
        tc_fence_before();
        mbar_arrive(&ctl->dp_loaded);  // dP of the next tile may overwrite these columns now
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          dpk[i >> 1] = pack2<kBf16>(pr[i] * (__uint_as_float(d0[i]) - delta_r),
                                     pr[i + 1] * (__uint_as_float(d0[i + 1]) - delta_r));
          dpk[16 + (i >> 1)] = pack2<kBf16>(pr[i + 32] * (__uint_as_float(d1[i]) - delta_r),
                                            pr[i + 33] * (__uint_as_float(d1[i + 1]) - delta_r));
        }
      }
      // dS (16-bit) goes over the S columns: both warps of this lane quadrant must have read S
      bar_sync_pair(1 + quad);
      tmem_st32(tSj + half * 32, dpk);
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(&ctl->ds_ready);
      cursor_next<kTile>(geom, p.span_pos, p.span_len, cur, j + 1 < n_tiles);
    }

    // epilogue: dQ * softmax_scale -> dq
    if (ok && n_tiles > 0) ok = mbar_wait(&ctl->done, 0, err, kErrWaitEpilogue);
    ok = __all_sync(0xffffffffu, ok);
    tc_fence_after();
    if (ok && ctl->err == 0) {
      uint16_t* drow = reinterpret_cast<uint16_t*>(p.dq) + b * p.dq_sb + static_cast<long long>(row0 + row) * p.dq_st +
                       h * p.dq_sh + half * 64;
      const float mul = p.scale;
#pragma unroll 1
      for (int c = 0; c < 2; ++c) {
        uint32_t r[32];
        if (n_tiles > 0) {
          tmem_ld32(tDQ + lane_off + half * 64 + c * 32, r);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) r[i] = 0u;
        }
        if (valid) {
          uint4* dst = reinterpret_cast<uint4*>(drow + c * 32);
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

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, kDqTmemCols);
  }
  if (threadIdx.x == 0 && ctl->err != 0) atomicCAS(p.status, 0, ctl->err);
}

}  // namespace

int launch_dq(const BwdKernelParams& kp, int dtype, cudaStream_t stream) {
  const int n_q_tiles = (kp.q_len + kTile - 1) / kTile;
  const long long n_cta = static_cast<long long>(n_q_tiles) * kp.hq * kp.batch;
  if (n_cta <= 0) return RSWA_OK;
  if (n_cta > 0x7fffffffLL) {
    set_error("rswa_bwd: too many query tiles (%lld)", n_cta);
    return RSWA_E_ARG;
  }
  auto kern = dtype == RSWA_DTYPE_BF16 ? rswa_dq_kernel<true> : rswa_dq_kernel<false>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kDqSmemBytes);
  if (e != cudaSuccess) {
    set_error("rswa_bwd(dq): cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    return RSWA_E_CUDA;
  }
  kern<<<static_cast<unsigned>(n_cta), kDqThreads, kDqSmemBytes, stream>>>(kp, n_q_tiles);
  e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_error("rswa_bwd(dq): launch: %s", cudaGetErrorString(e));
    return RSWA_E_CUDA;
  }
  return RSWA_OK;
}

}  // namespace rswa
