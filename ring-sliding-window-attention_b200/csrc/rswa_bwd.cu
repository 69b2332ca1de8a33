// dK/dV kernel: the key-stationary half of the backward pass.
//
// One CTA owns a 128-key tile of one KV head and walks every query tile (and every query head of
// the group) that can see it.  The products run in the transposed (key-major) form so that P and
// dS feed the next MMA as the A operand straight from tensor memory:
//
//   S^T  = K Q^T          A = K   (smem, K-major)     B = Q   (smem, K-major)
//   dP^T = V dO^T         A = V   (smem, K-major)     B = dO  (smem, K-major)
//   P^T  = exp2(S^T * scale_log2 - lse2),   dS^T = P^T * (dP^T - delta)      (8 compute warps)
//   dV  += P^T dO         A = P^T (TMEM)              B = dO  (smem, MN-major)
//   dK  += dS^T Q         A = dS^T(TMEM)              B = Q   (smem, MN-major)
//
// dK and dV stay in TMEM for the whole CTA (summed over the query heads of the group) and are
// written once.  dQ is the business of the query-stationary kernel (rswa_dq.cu), so nothing is
// reduced through global memory.  P is recomputed from the saved log-sum-exp, and delta is
// rowsum(dO * O), which is what makes a per-span backward against the FINAL out/lse exact (the
// property the reference's per-hop backward relies on, ring_swa/ops/attn.py:63-126).
//
// Pipeline: one thread issues every product, in the order  dV(i), dK(i), dP^T(i+1), S^T(i+2)  once
// P^T | dS^T of query tile i are in tensor memory: dP^T(i+1) overwrites their columns, which issue
// order makes safe without a wait, and S^T(i+2) fills the tensor pipe while the compute warps turn
// dP^T(i+1) into dS^T(i+1).  The exponentials of tile i+1 run off that critical loop.  Q tiles travel
// through a 3-stage ring (they are needed two tiles ahead), dO tiles through a 2-stage ring.
// TMEM columns: [0,128) dK, [128,256) dV, [256,384) S^T, [384,512) dP^T, over which each compute
// warp writes P^T and dS^T of the 64 query columns it has just read (P^T in the first 32 of its 64
// columns, dS^T in the other 32), handed over in two chunks of 32 queries.  dK and dV leave through
// shared memory as whole row segments.
#include "rswa_common.cuh"
#include "tc05.cuh"

namespace rswa {
using namespace tc05;

RSWA_TRACE_DECL(bwd)

namespace {

constexpr int kBwdThreads = 384;  // warp 0 TMA, warp 1 MMA, warps 2-3 idle, warps 4-11 compute
constexpr int kMmaPollNs = 0;  // the MMA-issuing threads poll without back-off (they are on the critical path)
constexpr int kBwdTmemCols = 512;
constexpr int kComputeThreads = 256;
constexpr int kQStages = 3;
#ifndef RSWA_BWD_POLY
#define RSWA_BWD_POLY 1
#endif
constexpr bool kBwdPoly = RSWA_BWD_POLY != 0;  // a quarter of the exponentials on the FMA pipe

struct BwdCtl {
  uint64_t kv_full, q_full[kQStages], q_free[kQStages], do_full[2], do_free[2];
  uint64_t s_ready, s_loaded, dp_ready, pds_ready[2], done;
  uint32_t tmem_base;
  int err;
  int qt_first, n_qt;
};

// K, V, 3 x Q, 2 x dO  +  3 lse2 rows + 2 delta rows  +  control
constexpr int kBwdSmemTiles = 7 * kTileBytes;
constexpr int kRowBytes = kTile * 4;
constexpr int kBwdSmemBytes = kBwdSmemTiles + (kQStages + 2) * kRowBytes + 256;
constexpr uint32_t kStageTxBytes = kTileBytes + kRowBytes;
static_assert(sizeof(BwdCtl) <= 256, "control block too large");
static_assert(kBwdSmemBytes <= 232448, "shared memory budget");


// kPlain: one KV span, no packed sequences, no sink tokens, 16-bit gradients (the plain sliding window
// of one GPU).  The SM's instruction cache holds 32 KB and every CTA runs through set-up, loop and
// epilogue once, so what such a call cannot need is compiled out of its variant.
template <bool kBf16, bool kPlain>
__global__ void __launch_bounds__(kBwdThreads, 1)
rswa_bwd_kernel(const __grid_constant__ BwdKernelParams p, int total_tiles) {
  const int* const cu_seq = kPlain ? nullptr : p.cu;
  const int n_seqs = kPlain ? 0 : p.n_seqs;
  const int n_spans = kPlain ? 1 : p.n_spans;
  const int n_sink = kPlain ? 0 : p.n_sink;
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* sK = smem;
  uint8_t* sV = smem + kTileBytes;
  uint8_t* sQ = smem + 2 * kTileBytes;   // three stages
  uint8_t* sDO = smem + 5 * kTileBytes;  // two stages
  float* sLse = reinterpret_cast<float*>(smem + kBwdSmemTiles);  // [3][128], travels with Q
  float* sDelta = sLse + kQStages * kTile;                       // [2][128], travels with dO
  BwdCtl* ctl = reinterpret_cast<BwdCtl*>(smem + kBwdSmemTiles + (kQStages + 2) * kRowBytes);

  RSWA_TRC(bwd, threadIdx.x == 0, 1920);
  // Has a device-side error already been reported on this stream?  Then this CTA does no work (no
  // further time-outs piled on the first).  The word is read now and looked at after the set-up
  // below, so that its latency is not paid at the head of every CTA.
  int prior = 0;
  if (threadIdx.x == 0) {
    prior = *reinterpret_cast<volatile int*>(p.status);
    prefetch_tmap(&p.q_map);
    prefetch_tmap(&p.do_map);
  }

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // work item: batch row fastest, then KV head, then key tile (tiles of the first span first)
  int idx = blockIdx.x;
  const int b = idx % p.batch;
  idx /= p.batch;
  const int hk = idx % p.hkv;
  const int kt_g = idx / p.hkv;
  int sp = 0;
  while (sp + 1 < n_spans && kt_g >= p.span_tile0[sp + 1]) ++sp;
  const int kt = kt_g - p.span_tile0[sp];
  const int key0 = kt * kTile;  // token offset inside the span
  const int n_valid_k = min(kTile, p.span_len[sp] - key0);
  const int t0 = p.span_pos[sp] + key0;
  const int group = p.hq / p.hkv;
  const int q_end_pos = p.q_pos_start + p.q_len;  // exclusive

  if (threadIdx.x == 0) {
    mbar_init(&ctl->kv_full, 1);
    for (int i = 0; i < kQStages; ++i) {
      mbar_init(&ctl->q_full[i], 1);
      mbar_init(&ctl->q_free[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&ctl->do_full[i], 1);
      mbar_init(&ctl->do_free[i], 1);
    }
    mbar_init(&ctl->s_ready, 1);
    mbar_init(&ctl->s_loaded, kComputeThreads / 32);  // one arrival per compute warp
    mbar_init(&ctl->dp_ready, 1);
    mbar_init(&ctl->pds_ready[0], kComputeThreads / 32);  // one arrival per compute warp and chunk of 32 queries
    mbar_init(&ctl->pds_ready[1], kComputeThreads / 32);
    mbar_init(&ctl->done, 1);
    mbar_fence_init();
    // K and V of this tile depend on nothing computed below: they are on their way while the rest
    // of the set-up runs (the CTA waits for them before it exits even if it has no work)
    mbar_expect_tx(&ctl->kv_full, 2 * kTileBytes);
    tma_load_4d(sK, &p.k_map[sp], &ctl->kv_full, 0, hk, key0, b);
    tma_load_4d(sK + kBoxBytes, &p.k_map[sp], &ctl->kv_full, 64, hk, key0, b);
    tma_load_4d(sV, &p.v_map[sp], &ctl->kv_full, 0, hk, key0, b);
    tma_load_4d(sV + kBoxBytes, &p.v_map[sp], &ctl->kv_full, 64, hk, key0, b);
    ctl->err = (smem_u32(smem) & 1023u) ? 199 : prior;
    // query tiles that can see at least one key of this tile
    const int t_last = t0 + n_valid_k - 1;
    int s_last, e_last;
    seq_of(cu_seq, n_seqs, t_last, s_last, e_last);
    int pmax;
    if (n_sink > 0 && s_last + n_sink > t0) {
      pmax = e_last - 1;  // the tile holds a sink token: every later query of that sequence
    } else {
      pmax = (e_last - 1 - t_last > p.window) ? t_last + p.window : e_last - 1;
    }
    const int q_lo = max(t0, p.q_pos_start);
    const int q_hi = min(pmax, q_end_pos - 1);
    if (q_lo <= q_hi) {
      ctl->qt_first = (q_lo - p.q_pos_start) / kTile;
      ctl->n_qt = (q_hi - p.q_pos_start) / kTile - ctl->qt_first + 1;
      if (ctl->err == 0) {
        // the first query tile's Q / lse and dO / delta are on their way before the CTA has finished its
        // set-up (the producer below continues with the second)
        const int h = hk * group, row0 = ctl->qt_first * kTile;
        const long long roff = b * p.d_sb + h * p.d_sh + row0;
        mbar_expect_tx(&ctl->q_full[0], kStageTxBytes);
        tma_load_4d(sQ, &p.q_map, &ctl->q_full[0], 0, h, row0, b);
        tma_load_4d(sQ + kBoxBytes, &p.q_map, &ctl->q_full[0], 64, h, row0, b);
        bulk_load_1d(sLse, p.lse2 + roff, kRowBytes, &ctl->q_full[0]);
        mbar_expect_tx(&ctl->do_full[0], kStageTxBytes);
        tma_load_4d(sDO, &p.do_map, &ctl->do_full[0], 0, h, row0, b);
        tma_load_4d(sDO + kBoxBytes, &p.do_map, &ctl->do_full[0], 64, h, row0, b);
        bulk_load_1d(sDelta, p.delta + roff, kRowBytes, &ctl->do_full[0]);
      }
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

  RSWA_TRC(bwd, threadIdx.x == 0, 1921);
  const uint32_t tmem = ctl->tmem_base;
  const uint32_t tDK = tmem, tDV = tmem + 128, tS = tmem + 256, tB = tmem + 384;
  volatile int* err = &ctl->err;
  const int qt_first = ctl->qt_first;
  const int n_qt = (ctl->err != 0) ? 0 : ctl->n_qt;
  const int n_iter = n_qt * group;
  constexpr uint32_t kTile16 = kTileBytes >> 4;

  if (warp < 4) {
    setmaxnreg_dec<80>();
    if (warp == 0 && lane == 0 && n_iter > 0) {
      // ------------------------------------------------------------------ TMA producer
      bool ok = true;
      for (int it = 1; it < n_iter && ok; ++it) {  // (the first tile's loads were issued during the set-up)
        const int sq = it % kQStages, sd = it & 1;
        const int h = hk * group + it / n_qt;
        const int row0 = (qt_first + it % n_qt) * kTile;
        const long long roff = b * p.d_sb + h * p.d_sh + row0;
        if (it >= kQStages) ok = mbar_wait<200>(&ctl->q_free[sq], ((it / kQStages) - 1) & 1, err, kErrWaitProducer);
        if (!ok) break;
        mbar_expect_tx(&ctl->q_full[sq], kStageTxBytes);
        tma_load_4d(sQ + sq * kTileBytes, &p.q_map, &ctl->q_full[sq], 0, h, row0, b);
        tma_load_4d(sQ + sq * kTileBytes + kBoxBytes, &p.q_map, &ctl->q_full[sq], 64, h, row0, b);
        bulk_load_1d(sLse + sq * kTile, p.lse2 + roff, kRowBytes, &ctl->q_full[sq]);
        if (it >= 2) ok = mbar_wait<200>(&ctl->do_free[sd], ((it >> 1) - 1) & 1, err, kErrWaitProducer);
        if (!ok) break;
        mbar_expect_tx(&ctl->do_full[sd], kStageTxBytes);
        tma_load_4d(sDO + sd * kTileBytes, &p.do_map, &ctl->do_full[sd], 0, h, row0, b);
        tma_load_4d(sDO + sd * kTileBytes + kBoxBytes, &p.do_map, &ctl->do_full[sd], 64, h, row0, b);
        bulk_load_1d(sDelta + sd * kTile, p.delta + roff, kRowBytes, &ctl->do_full[sd]);
      }
    } else if (warp == 1 && n_iter > 0 && elect_one()) {
      // ------------------------------------------------------------------ MMA issuer
      // ONE elected thread issues every product and does all the waiting for them (a warp-wide vote
      // behind each wait costs more than it saves).  Steady-state order, once P^T | dS^T of tile i is
      // in tensor memory:   dV(i), dK(i), dP^T(i+1), S^T(i+2).
      // dP^T(i+1) overwrites the columns that hold P^T | dS^T of tile i; products of one thread execute
      // in issue order, so it needs no wait for dV(i) and dK(i).  S^T(i+2) goes last: nothing on the
      // loop that bounds the kernel needs it soon, and there it fills the tensor pipe while the compute
      // warps turn dP^T(i+1) into dS^T(i+1) (issued from a second thread it interleaved with the three
      // products ahead of it and delayed them by a third).
      constexpr int bf = kBf16 ? 1 : 0;
      constexpr uint32_t id_kk = idesc_f16(128, 128, bf, 0, 0);  // both operands K-major
      constexpr uint32_t id_tn = idesc_f16(128, 128, bf, 0, 1);  // A from TMEM, B MN-major
      const uint64_t dK = smem_desc_sw128(smem_u32(sK), 16, 1024);
      const uint64_t dV = smem_desc_sw128(smem_u32(sV), 16, 1024);
      const uint64_t dQk = smem_desc_sw128(smem_u32(sQ), 16, 1024);
      const uint64_t dQm = smem_desc_sw128(smem_u32(sQ), kBoxBytes, 1024);
      const uint64_t dDOk = smem_desc_sw128(smem_u32(sDO), 16, 1024);
      const uint64_t dDOm = smem_desc_sw128(smem_u32(sDO), kBoxBytes, 1024);
      // One loop turn per query tile and ONE copy of each product's code; the turns -2 and -1 fill the
      // pipeline (S^T(0); then dP^T(0), S^T(1)).
      bool ok = mbar_wait<kMmaPollNs>(&ctl->kv_full, 0, err, kErrWaitMma);
      for (int it = -2; it < n_iter && ok; ++it) {
        if (it >= 0) {
          const uint64_t dDOs = dDOm + (it & 1) * kTile16;
          const uint64_t dQs = dQm + (it % kQStages) * kTile16;
#pragma unroll 1
          for (int ch = 0; ch < 2; ++ch) {
            // P^T | dS^T arrive in two chunks: every compute warp's first 32 query columns (k-steps
            // 0, 1, 4, 5 of the 128 queries), then its other 32 (k-steps 2, 3, 6, 7)
            ok = mbar_wait<kMmaPollNs>(&ctl->pds_ready[ch], it & 1, err, kErrWaitMma);
            if (!ok) break;
            RSWA_TRC(bwd, it < 32 && ch == 0, it * 32 + 8);
            tc_fence_after();
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {  // dV += P^T dO
              const int k = (kk >> 1) * 4 + 2 * ch + (kk & 1);
              mma_ts(tDV, tB + (k >> 2) * 64 + (k & 3) * 8, dDOs + k * 128, id_tn, (it > 0 || ch > 0 || kk > 0) ? 1u : 0u);
            }
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {  // dK += dS^T Q
              const int k = (kk >> 1) * 4 + 2 * ch + (kk & 1);
              mma_ts(tDK, tB + (k >> 2) * 64 + 32 + (k & 3) * 8, dQs + k * 128, id_tn, (it > 0 || ch > 0 || kk > 0) ? 1u : 0u);
            }
          }
          if (!ok) break;
          mma_commit(&ctl->do_free[it & 1]);         // (dP^T of this tile, the stage's other reader, was issued before)
          mma_commit(&ctl->q_free[it % kQStages]);   // (S^T of this tile, the stage's other reader, was issued before)
          RSWA_TRC(bwd, it < 32, it * 32 + 9);
        }
        if (it + 1 >= 0 && it + 1 < n_iter) {
          // dP^T of the next query tile (it overwrites P^T | dS^T of this one: ordered behind their readers above)
          const int t = it + 1, sd = t & 1;
          ok = mbar_wait<kMmaPollNs>(&ctl->do_full[sd], (t >> 1) & 1, err, kErrWaitMma);
          if (!ok) break;
          tc_fence_after();
          const uint64_t dDOs = dDOk + sd * kTile16;
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const uint32_t off = ((k >> 2) * kBoxBytes + (k & 3) * 32) >> 4;
            mma_ss(tB, dV + off, dDOs + off, id_kk, k > 0 ? 1u : 0u);
          }
          mma_commit(&ctl->dp_ready);
        }
        RSWA_TRC(bwd, it >= 0 && it < 32, it * 32 + 11);
        if (it + 2 < n_iter) {
          // S^T of the query tile after next, once the compute warps hold the tile before it in registers
          const int t = it + 2, sq = t % kQStages;
          ok = mbar_wait<kMmaPollNs>(&ctl->q_full[sq], (t / kQStages) & 1, err, kErrWaitMma);
          if (ok && t > 0) ok = mbar_wait<kMmaPollNs>(&ctl->s_loaded, (t - 1) & 1, err, kErrWaitMma);
          if (!ok) break;
          tc_fence_after();
          const uint64_t dQs = dQk + sq * kTile16;
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const uint32_t off = ((k >> 2) * kBoxBytes + (k & 3) * 32) >> 4;
            mma_ss(tS, dK + off, dQs + off, id_kk, k > 0 ? 1u : 0u);
          }
          mma_commit(&ctl->s_ready);
        }
      }
      if (ok) mma_commit(&ctl->done);
    }
  } else {
    // -------------------------------------------------------------------- compute warps
    setmaxnreg_inc<208>();  // 128 x 80 + 256 x 208 <= 384 x 168 (the launch allocation)
    const int quad = warp & 3;
    const int half = (warp - 4) >> 2;            // which 64 query columns this warp handles
    const int row = quad * 32 + lane;            // key row
    const uint32_t lane_off = static_cast<uint32_t>(quad * 32) << 16;
    const bool valid_k = row < n_valid_k;
    const int t = valid_k ? t0 + row : 0x7fffffff;
    int p_hi = -1;
    if (valid_k) {
      int s_t, e_t;
      seq_of(cu_seq, n_seqs, t, s_t, e_t);
      const bool is_sink = t < s_t + n_sink;
      p_hi = (is_sink || e_t - 1 - t <= p.window) ? e_t - 1 : t + p.window;
      p_hi = min(p_hi, q_end_pos - 1);
    }
    const float sl2 = p.scale_log2;
    bool ok = true;

    for (int it = 0; it < n_iter && ok; ++it) {
      const int qrow0 = (qt_first + it % n_qt) * kTile;
      const int pq0 = p.q_pos_start + qrow0;
      const float* lse_s = sLse + (it % kQStages) * kTile + half * 64;
      const float* del_s = sDelta + (it & 1) * kTile + half * 64;
      const bool full = (pq0 >= t) && (pq0 + kTile - 1 <= p_hi);
      const bool masked = !__all_sync(0xffffffffu, full);

      // P^T from S^T (the lse2 row of this stage landed together with Q, before S^T was issued)
      ok = mbar_wait(&ctl->s_ready, it & 1, err, kErrWaitSoftmax);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      RSWA_TRC(bwd, warp == 4 && lane == 0 && it < 32, it * 32 + 0);
      tc_fence_after();
      float pr[64];
      {
        uint32_t s0[32], s1[32];
        tmem_ld32(tS + lane_off + half * 64, s0);
        tmem_ld32(tS + lane_off + half * 64 + 32, s1);
        tmem_ld_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&ctl->s_loaded);  // S^T of the next query tile may overwrite these columns now
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
          const float4 la = *reinterpret_cast<const float4*>(lse_s + i);
          const float4 lb = *reinterpret_cast<const float4*>(lse_s + i + 32);
          const float xa0 = fmaf(__uint_as_float(s0[i + 0]), sl2, -la.x), xa1 = fmaf(__uint_as_float(s0[i + 1]), sl2, -la.y);
          const float xa2 = fmaf(__uint_as_float(s0[i + 2]), sl2, -la.z), xa3 = fmaf(__uint_as_float(s0[i + 3]), sl2, -la.w);
          const float xb0 = fmaf(__uint_as_float(s1[i + 0]), sl2, -lb.x), xb1 = fmaf(__uint_as_float(s1[i + 1]), sl2, -lb.y);
          const float xb2 = fmaf(__uint_as_float(s1[i + 2]), sl2, -lb.z), xb3 = fmaf(__uint_as_float(s1[i + 3]), sl2, -lb.w);
          // one pair in four goes through the FMA pipe instead of the special-function unit
          pr[i + 0] = ex2f(xa0), pr[i + 1] = ex2f(xa1);
          pr[i + 32] = ex2f(xb0), pr[i + 33] = ex2f(xb1);
          if (kBwdPoly && (i & 4)) {
            const float2 ea = ex2_poly2(make_float2(xa2, xa3)), eb = ex2_poly2(make_float2(xb2, xb3));
            pr[i + 2] = ea.x, pr[i + 3] = ea.y, pr[i + 34] = eb.x, pr[i + 35] = eb.y;
          } else {
            pr[i + 2] = ex2f(xa2), pr[i + 3] = ex2f(xa3);
            pr[i + 34] = ex2f(xb2), pr[i + 35] = ex2f(xb3);
          }
        }
      }
      if (masked) {
#pragma unroll
        for (int i = 0; i < 64; ++i) {
          const int pq = pq0 + half * 64 + i;
          pr[i] = (pq >= t && pq <= p_hi) ? pr[i] : 0.f;
        }
      }
      // Everything that does not need dP^T happens before the wait for it (the wait is on the loop
      // that bounds the kernel): P^T is packed, and -P^T * delta is formed so that one FMA per
      // element remains afterwards: dS^T = P^T * dP^T - P^T * delta.
      uint32_t ppk[32];
#pragma unroll
      for (int i = 0; i < 64; i += 2) ppk[i >> 1] = pack2<kBf16>(pr[i], pr[i + 1]);
      // the delta row travels with the dO stage: it must have landed before it is read (the MMA
      // warps wait for the stage before dP^T, the compute warps have not waited for anything of it yet)
      ok = mbar_wait(&ctl->do_full[it & 1], (it >> 1) & 1, err, kErrWaitSoftmax);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      float npd[64];
#pragma unroll
      for (int i = 0; i < 32; i += 4) {
        const float4 da = *reinterpret_cast<const float4*>(del_s + i);
        const float4 db = *reinterpret_cast<const float4*>(del_s + i + 32);
        npd[i + 0] = -pr[i + 0] * da.x, npd[i + 1] = -pr[i + 1] * da.y;
        npd[i + 2] = -pr[i + 2] * da.z, npd[i + 3] = -pr[i + 3] * da.w;
        npd[i + 32] = -pr[i + 32] * db.x, npd[i + 33] = -pr[i + 33] * db.y;
        npd[i + 34] = -pr[i + 34] * db.z, npd[i + 35] = -pr[i + 35] * db.w;
      }
      RSWA_TRC(bwd, warp == 4 && lane == 0 && it < 32, it * 32 + 1);
      ok = mbar_wait(&ctl->dp_ready, it & 1, err, kErrWaitSoftmax);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      RSWA_TRC(bwd, warp == 4 && lane == 0 && it < 32, it * 32 + 2);
      tc_fence_after();
      {
        // every dP^T column of this warp is read before any is overwritten
        uint32_t d[64];
        tmem_ld32(tB + lane_off + half * 64, *reinterpret_cast<uint32_t(*)[32]>(&d[0]));
        tmem_ld32(tB + lane_off + half * 64 + 32, *reinterpret_cast<uint32_t(*)[32]>(&d[32]));
        tmem_ld_wait();
        // P^T and dS^T (16-bit) go over the very dP^T columns this warp has just read, so no other
        // warp has to be waited for: columns [64 half, +32) hold P^T, [64 half + 32, +32) hold dS^T.
        // They are handed over in two chunks of 32 queries, so that the products of the first chunk
        // run while the second is still being formed.
#pragma unroll
        for (int ch = 0; ch < 2; ++ch) {
          uint32_t pp[16], dd[16];
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const int e = ch * 32 + i;
            pp[i >> 1] = ppk[e >> 1];
            dd[i >> 1] = pack2<kBf16>(fmaf(pr[e], __uint_as_float(d[e]), npd[e]),
                                      fmaf(pr[e + 1], __uint_as_float(d[e + 1]), npd[e + 1]));
          }
          tmem_st16(tB + lane_off + half * 64 + ch * 16, pp);
          tmem_st16(tB + lane_off + half * 64 + 32 + ch * 16, dd);
          tmem_st_wait();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&ctl->pds_ready[ch]);
        }
      }
      RSWA_TRC(bwd, warp == 4 && lane == 0 && it < 32, it * 32 + 3);
    }

    // epilogue: dK (scaled) and dV for this key tile
    RSWA_TRC(bwd, warp == 4 && lane == 0, 1922);
    if (ok && n_iter > 0) ok = mbar_wait(&ctl->done, 0, err, kErrWaitEpilogue);
    RSWA_TRC(bwd, warp == 4 && lane == 0, 1923);
    ok = __all_sync(0xffffffffu, ok);
    tc_fence_after();
    if (ok && ctl->err == 0) {
      // Each thread holds 64 columns of one key row; stored from registers that would be 32 different
      // lines per instruction.  The rows therefore pass through shared memory (this warp's 8 KB of
      // the Q ring, free now that every product has completed; 16-byte chunks XOR-swizzled by row)
      // and leave as whole 128- or 256-byte row segments, several rows per instruction.
      uint8_t* stage = sQ + (warp - 4) * 8192;
      const int n_rows = n_valid_k - quad * 32;  // key rows of this warp that exist
      const long long off0 = b * p.dkv_sb[sp] + static_cast<long long>(key0 + quad * 32) * p.dkv_st[sp] +
                             hk * p.dkv_sh[sp] + half * 64;
      const long long rst = p.dkv_st[sp];
      const bool f32 = !kPlain && p.grad_fp32[sp] != 0;
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
          if (f32) {
#pragma unroll
            for (int v = 0; v < 8; ++v) {
              const float4 o = make_float4(__uint_as_float(r[v * 4]) * mul, __uint_as_float(r[v * 4 + 1]) * mul,
                                           __uint_as_float(r[v * 4 + 2]) * mul, __uint_as_float(r[v * 4 + 3]) * mul);
              *reinterpret_cast<float4*>(stage + lane * 256 + (((c * 8 + v) ^ (lane & 15)) << 4)) = o;
            }
          } else {
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              uint4 o;
              o.x = pack2<kBf16>(__uint_as_float(r[v * 8 + 0]) * mul, __uint_as_float(r[v * 8 + 1]) * mul);
              o.y = pack2<kBf16>(__uint_as_float(r[v * 8 + 2]) * mul, __uint_as_float(r[v * 8 + 3]) * mul);
              o.z = pack2<kBf16>(__uint_as_float(r[v * 8 + 4]) * mul, __uint_as_float(r[v * 8 + 5]) * mul);
              o.w = pack2<kBf16>(__uint_as_float(r[v * 8 + 6]) * mul, __uint_as_float(r[v * 8 + 7]) * mul);
              *reinterpret_cast<uint4*>(stage + lane * 128 + (((c * 4 + v) ^ (lane & 7)) << 4)) = o;
            }
          }
        }
        __syncwarp();
        if (f32) {
          const int ch = lane & 15;
#pragma unroll 4
          for (int i = 0; i < 16; ++i) {  // two 256-byte row segments per instruction
            const int rr = 2 * i + (lane >> 4);
            const float4 o = *reinterpret_cast<const float4*>(stage + rr * 256 + ((ch ^ (rr & 15)) << 4));
            if (rr < n_rows) *reinterpret_cast<float4*>(static_cast<float*>(base) + off0 + rr * rst + ch * 4) = o;
          }
        } else {
          const int ch = lane & 7;
#pragma unroll 4
          for (int i = 0; i < 8; ++i) {  // four 128-byte row segments per instruction
            const int rr = 4 * i + (lane >> 3);
            const uint4 o = *reinterpret_cast<const uint4*>(stage + rr * 128 + ((ch ^ (rr & 7)) << 4));
            if (rr < n_rows) *reinterpret_cast<uint4*>(static_cast<uint16_t*>(base) + off0 + rr * rst + ch * 8) = o;
          }
        }
        __syncwarp();  // the staging rows are rewritten for dV
      }
    }
  }

  RSWA_TRC(bwd, warp == 4 && lane == 0, 1924);
  // no product waited for K and V: their copy must still have landed before the CTA goes away
  if (threadIdx.x == 0 && n_iter == 0) mbar_wait<200>(&ctl->kv_full, 0, err, kErrWaitProducer);
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, kBwdTmemCols);
  }
  RSWA_TRC(bwd, threadIdx.x == 0, 1925);
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
  const bool plain = kp.n_spans == 1 && kp.cu == nullptr && kp.n_sink == 0 && kp.grad_fp32[0] == 0;
  const int variant = (dtype == RSWA_DTYPE_BF16 ? 1 : 0) + (plain ? 2 : 0);
  using Kern = void (*)(const BwdKernelParams, int);
  static const Kern kerns[4] = {rswa_bwd_kernel<false, false>, rswa_bwd_kernel<true, false>,
                                rswa_bwd_kernel<false, true>, rswa_bwd_kernel<true, true>};
  const Kern kern = kerns[variant];
  // (the attribute is a property of the function on a device: set once per kernel variant and device)
  static bool attr_set[4][64] = {{false}};
  int dev_id = 0;
  cudaError_t e = cudaGetDevice(&dev_id);
  if (e == cudaSuccess && (dev_id < 0 || dev_id >= 64 || !attr_set[variant][dev_id])) {
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kBwdSmemBytes);
    if (e == cudaSuccess && dev_id >= 0 && dev_id < 64) attr_set[variant][dev_id] = true;
  }
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
