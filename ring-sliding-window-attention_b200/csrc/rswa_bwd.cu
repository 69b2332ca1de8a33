// dK/dV kernel: the key-stationary half of the backward pass.
//
// A work item is a 128-key tile of one KV head; the CTA that takes it walks every query tile (and every
// query head of the group) that can see it.  The products run in the transposed (key-major) form so
// that P and dS feed the next MMA as the A operand straight from tensor memory:
//
//   S^T  = K Q^T          A = K   (smem, K-major)     B = Q   (smem, K-major)
//   dP^T = V dO^T         A = V   (smem, K-major)     B = dO  (smem, K-major)
//   P^T  = exp2(S^T * scale_log2 - lse2),   dS^T = P^T * (dP^T - delta)      (8 compute warps)
//   dV  += P^T dO         A = P^T (TMEM)              B = dO  (smem, MN-major)
//   dK  += dS^T Q         A = dS^T(TMEM)              B = Q   (smem, MN-major)
//
// dK and dV stay in TMEM for the whole item (summed over the query heads of the group) and are written
// once.  dQ is the business of the query-stationary kernel (rswa_dq.cu), so nothing is reduced through
// global memory.  P is recomputed from the saved log-sum-exp, and delta is rowsum(dO * O), which is
// what makes a per-span backward against the FINAL out/lse exact (the property the reference's per-hop
// backward relies on, ring_swa/ops/attn.py:63-126).
//
// The kernel is persistent: one CTA per SM takes items from a counter in global memory, and every
// pipeline (Q / dO rings, barrier phases) keeps running across item boundaries.  K and V have one buffer
// each; they are reloaded as soon as the item's last S^T and dP^T products have been issued, i.e. while
// its last two query tiles still run, and the item's dK / dV are read out and stored behind the first
// exponentials of the next item.  (A one-shot CTA per key tile spent 4 100 cycles of a 34 500-cycle
// life waiting for its first loads, and its epilogue and the launch gap were not overlapped either.)
//
// Pipeline: one thread issues every product, in the order  dV(i), dK(i), dP^T(i+1), S^T(i+2)  once
// P^T | dS^T of query tile i are in tensor memory: dP^T(i+1) overwrites their columns, which issue
// order makes safe without a wait, and S^T(i+2) fills the tensor pipe while the compute warps turn
// dP^T(i+1) into dS^T(i+1).  The exponentials of tile i+1 run off that critical loop.  Q tiles travel
// through a 3-stage ring (they are needed two tiles ahead), dO tiles through a 2-stage ring.
// TMEM columns: [0,128) dK, [128,256) dV, [256,384) S^T, [384,512) dP^T, over which each compute
// warp writes P^T and dS^T of the 64 query columns it has just read (P^T in the first 32 of its 64
// columns, dS^T in the other 32), handed over in two chunks of 32 queries.  dK and dV leave with
// 32-byte stores from registers (a thread owns 64 consecutive columns of one key row).
#include "rswa_common.cuh"
#include "tc05.cuh"

namespace rswa {
using namespace tc05;

RSWA_TRACE_DECL(bwd)
#ifndef RSWA_TRACE_G0
#define RSWA_TRACE_G0 100
#endif
#define BWD_TRC(cond, g, s) RSWA_TRC(bwd, (cond) && (g) >= RSWA_TRACE_G0 && (g) < RSWA_TRACE_G0 + 32, ((g) - RSWA_TRACE_G0) * 32 + (s))

namespace {

constexpr int kBwdThreads = 384;  // warp 0 TMA, warp 1 MMA, warps 2-3 idle, warps 4-11 compute
constexpr int kMmaPollNs = 0;  // the MMA-issuing threads poll without back-off (they are on the critical path)
constexpr int kBwdTmemCols = 512;
constexpr int kComputeThreads = 256;
constexpr int kQStages = 3;
#ifndef RSWA_BWD_POLY
#define RSWA_BWD_POLY 1
#endif
constexpr bool kBwdPoly = RSWA_BWD_POLY != 0;  // a quarter of the exponentials on the FMA pipe (worth 0.6 % here: two compute warps per scheduler need 1 024 cycles of the special-function unit per query tile)

// what every role needs to know about a work item (one key tile of one KV head), filled by the producer
struct BwdItemGeom {
  int valid;  // 0: no more work
  int b, hk, sp, key0, n_valid_k, t0, qt_first, n_qt;
};

struct BwdCtl {
  uint64_t kv_full, kv_free, q_full[kQStages], q_free[kQStages], do_full[2], do_free[2];
  uint64_t s_ready, s_loaded, dp_ready, pds_ready[2], done, acc_free;
  uint64_t geom_full[2], geom_free[2];
  uint32_t tmem_base;
  int err;
  BwdItemGeom geom[2];
};

// K, V, 3 x Q, 2 x dO  +  3 lse2 rows + 2 delta rows  +  control
constexpr int kBwdSmemTiles = 7 * kTileBytes;
constexpr int kRowBytes = kTile * 4;
constexpr int kBwdSmemBytes = kBwdSmemTiles + (kQStages + 2) * kRowBytes + 512;
constexpr uint32_t kStageTxBytes = kTileBytes + kRowBytes;
constexpr int kGeomUsers = 1 + kComputeThreads / 32;  // the MMA thread and one lane per compute warp
static_assert(sizeof(BwdCtl) <= 512, "control block too large");
static_assert(kBwdSmemBytes <= 232448, "shared memory budget");

// kPlain: one KV span, no packed sequences, no sink tokens, 16-bit gradients (the plain sliding window
// of one GPU): what such a call cannot need is compiled out of its variant (the SM's instruction
// cache holds 32 KB).
template <bool kBf16, bool kPlain>
__global__ void __launch_bounds__(kBwdThreads, 1)
rswa_bwd_kernel(const __grid_constant__ BwdKernelParams p, int n_items) {
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

  // a device-side error was already reported on this stream: do not pile further time-outs on it
  if (__syncthreads_or(*reinterpret_cast<volatile int*>(p.status) != 0)) return;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int group = p.hq / p.hkv;
  const int q_end_pos = p.q_pos_start + p.q_len;  // exclusive

  if (threadIdx.x == 0) {
    mbar_init(&ctl->kv_full, 1);
    mbar_init(&ctl->kv_free, 1);
    for (int i = 0; i < kQStages; ++i) {
      mbar_init(&ctl->q_full[i], 1);
      mbar_init(&ctl->q_free[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&ctl->do_full[i], 1);
      mbar_init(&ctl->do_free[i], 1);
      mbar_init(&ctl->pds_ready[i], kComputeThreads / 32);  // one arrival per compute warp and chunk of 32 queries
      mbar_init(&ctl->geom_full[i], 1);
      mbar_init(&ctl->geom_free[i], kGeomUsers);
    }
    mbar_init(&ctl->s_ready, 1);
    mbar_init(&ctl->s_loaded, kComputeThreads / 32);  // one arrival per compute warp
    mbar_init(&ctl->dp_ready, 1);
    mbar_init(&ctl->done, 1);
    mbar_init(&ctl->acc_free, kComputeThreads / 32);
    ctl->err = (smem_u32(smem) & 1023u) ? 199 : 0;
    mbar_fence_init();
    prefetch_tmap(&p.q_map);
    prefetch_tmap(&p.do_map);
  }
  if (warp == 1) {
    tmem_alloc(&ctl->tmem_base, kBwdTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();

  const uint32_t tmem = ctl->tmem_base;
  const uint32_t tDK = tmem, tDV = tmem + 128, tS = tmem + 256, tB = tmem + 384;
  volatile int* err = &ctl->err;
  const int n_work = (ctl->err != 0) ? 0 : n_items;
  constexpr uint32_t kTile16 = kTileBytes >> 4;

  if (warp < 4) {
    setmaxnreg_dec<80>();
    if (warp == 0 && lane == 0) {
      // ------------------------------------------------------------------ item geometry + TMA producer
      int gi = 0;  // query tiles loaded so far, all items (ring stages and barrier phases)
      int nk = 0;  // items with work so far
      for (int n = 0;; ++n) {
        const int slot = n & 1;
        if (n >= 2 && !mbar_wait<200>(&ctl->geom_free[slot], ((n >> 1) - 1) & 1, err, kErrWaitProducer)) break;
        BwdItemGeom* g = &ctl->geom[slot];
        // work item: batch row fastest, then KV head, then key tile (tiles of the first span first)
        // Items are handed out through a counter in global memory, in index order: a CTA that got a long
        // item (the key tile that holds a sink token is seen by every later query tile of its sequence)
        // or started late simply takes fewer.
        int idx = n_work > 0 ? atomicAdd(p.dkv_counter, 1) : n_work;
        if (idx >= n_work) {
          g->valid = 0;
          mbar_arrive(&ctl->geom_full[slot]);
          break;
        }
        const int b = idx % p.batch;
        idx /= p.batch;
        const int hk = idx % p.hkv;
        const int kt_g = idx / p.hkv;
        int sp = 0;
        while (sp + 1 < n_spans && kt_g >= p.span_tile0[sp + 1]) ++sp;
        const int key0 = (kt_g - p.span_tile0[sp]) * kTile;  // token offset inside the span
        const int n_valid_k = min(kTile, p.span_len[sp] - key0);
        const int t0 = p.span_pos[sp] + key0;
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
        int qt_first = 0, n_qt = 0;
        if (q_lo <= q_hi) {
          qt_first = (q_lo - p.q_pos_start) / kTile;
          n_qt = (q_hi - p.q_pos_start) / kTile - qt_first + 1;
        }
        g->valid = 1, g->b = b, g->hk = hk, g->sp = sp, g->key0 = key0, g->n_valid_k = n_valid_k, g->t0 = t0;
        g->qt_first = qt_first, g->n_qt = n_qt;
        mbar_arrive(&ctl->geom_full[slot]);
        if (n_qt == 0) continue;
        // K and V have one buffer each: the previous item's last S^T and dP^T products must have read them
        if (nk > 0 && !mbar_wait<200>(&ctl->kv_free, (nk - 1) & 1, err, kErrWaitProducer)) break;
        ++nk;
        mbar_expect_tx(&ctl->kv_full, 2 * kTileBytes);
        tma_load_4d(sK, &p.k_map[sp], &ctl->kv_full, 0, hk, key0, b);
        tma_load_4d(sK + kBoxBytes, &p.k_map[sp], &ctl->kv_full, 64, hk, key0, b);
        tma_load_4d(sV, &p.v_map[sp], &ctl->kv_full, 0, hk, key0, b);
        tma_load_4d(sV + kBoxBytes, &p.v_map[sp], &ctl->kv_full, 64, hk, key0, b);
        bool ok = true;
        for (int ih = 0; ih < group && ok; ++ih) {
          const int h = hk * group + ih;
#pragma unroll 1
          for (int iq = 0; iq < n_qt; ++iq, ++gi) {
            const int sq = gi % kQStages, sd = gi & 1;
            const int row0 = (qt_first + iq) * kTile;
            const long long roff = b * p.d_sb + h * p.d_sh + row0;
            if (gi >= kQStages) ok = mbar_wait<200>(&ctl->q_free[sq], ((gi / kQStages) - 1) & 1, err, kErrWaitProducer);
            if (!ok) break;
            mbar_expect_tx(&ctl->q_full[sq], kStageTxBytes);
            tma_load_4d(sQ + sq * kTileBytes, &p.q_map, &ctl->q_full[sq], 0, h, row0, b);
            tma_load_4d(sQ + sq * kTileBytes + kBoxBytes, &p.q_map, &ctl->q_full[sq], 64, h, row0, b);
            bulk_load_1d(sLse + sq * kTile, p.lse2 + roff, kRowBytes, &ctl->q_full[sq]);
            if (gi >= 2) ok = mbar_wait<200>(&ctl->do_free[sd], ((gi >> 1) - 1) & 1, err, kErrWaitProducer);
            if (!ok) break;
            mbar_expect_tx(&ctl->do_full[sd], kStageTxBytes);
            tma_load_4d(sDO + sd * kTileBytes, &p.do_map, &ctl->do_full[sd], 0, h, row0, b);
            tma_load_4d(sDO + sd * kTileBytes + kBoxBytes, &p.do_map, &ctl->do_full[sd], 64, h, row0, b);
            bulk_load_1d(sDelta + sd * kTile, p.delta + roff, kRowBytes, &ctl->do_full[sd]);
          }
        }
        if (!ok) break;
      }
    } else if (warp == 1 && elect_one()) {
      // ------------------------------------------------------------------ MMA issuer
      // ONE elected thread issues every product and does all the waiting for them (a warp-wide vote
      // behind each wait costs more than it saves).  Steady-state order, once P^T | dS^T of tile i is
      // in tensor memory:   dV(i), dK(i), dP^T(i+1), S^T(i+2).
      // dP^T(i+1) overwrites the columns that hold P^T | dS^T of tile i; products of one thread execute
      // in issue order, so it needs no wait for dV(i) and dK(i).  S^T(i+2) goes last: nothing on the
      // loop that bounds the kernel needs it soon, and there it fills the tensor pipe while the compute
      // warps turn dP^T(i+1) into dS^T(i+1).  The first S^T and dP^T of the NEXT item follow the last
      // dV / dK of this one directly: its K and V were loaded while this item's last tiles ran.
      constexpr int bf = kBf16 ? 1 : 0;
      constexpr uint32_t id_kk = idesc_f16(128, 128, bf, 0, 0);  // both operands K-major
      constexpr uint32_t id_tn = idesc_f16(128, 128, bf, 0, 1);  // A from TMEM, B MN-major
      const uint64_t dK = smem_desc_sw128(smem_u32(sK), 16, 1024);
      const uint64_t dV = smem_desc_sw128(smem_u32(sV), 16, 1024);
      const uint64_t dQk = smem_desc_sw128(smem_u32(sQ), 16, 1024);
      const uint64_t dQm = smem_desc_sw128(smem_u32(sQ), kBoxBytes, 1024);
      const uint64_t dDOk = smem_desc_sw128(smem_u32(sDO), 16, 1024);
      const uint64_t dDOm = smem_desc_sw128(smem_u32(sDO), kBoxBytes, 1024);
      int gbase = 0, nk = 0;  // query tiles of earlier items, items with work so far
      bool ok = true;
      for (int n = 0; ok; ++n) {
        const int slot = n & 1;
        ok = mbar_wait<kMmaPollNs>(&ctl->geom_full[slot], (n >> 1) & 1, err, kErrWaitMma);
        if (!ok || ctl->geom[slot].valid == 0) break;
        const int n_iter = ctl->geom[slot].n_qt * group;
        mbar_arrive(&ctl->geom_free[slot]);
        if (n_iter == 0) continue;
        ok = mbar_wait<kMmaPollNs>(&ctl->kv_full, nk & 1, err, kErrWaitMma);
        // one loop turn per query tile and ONE copy of each product's code; the turns -2 and -1 fill
        // the pipeline (S^T(0); then dP^T(0), S^T(1))
        // Every barrier is PROBED one block of products ahead of where it is needed (mbarrier.try_wait once,
        // the result looked at only after the block in between has been issued): this thread is the
        // longest chain of the CTA, and the round trip of a probe that finds its barrier complete, as it
        // nearly always does, otherwise stands between two blocks of products.  A probe that fails is
        // followed by the ordinary bounded wait.
        auto settle = [&](bool probed, uint64_t* bar, uint32_t parity) -> bool {
          return probed || mbar_wait<kMmaPollNs>(bar, parity, err, kErrWaitMma);
        };
        for (int it = -2; it < n_iter && ok; ++it) {
          const bool has_acc = it >= 0, has_dp = it + 1 >= 0 && it + 1 < n_iter, has_s = it + 2 < n_iter;
          const int g = gbase + it, tp = g + 1, ts = g + 2;
          const int sd = tp & 1, sq = ts % kQStages;
          bool pr_do = false, pr_q = false, pr_sl = false;
          if (has_acc) {
            const uint64_t dDOs = dDOm + (g & 1) * kTile16;
            const uint64_t dQs = dQm + (g % kQStages) * kTile16;
            const bool pr0 = mbar_try_wait(&ctl->pds_ready[0], g & 1);
            const bool pr1 = mbar_try_wait(&ctl->pds_ready[1], g & 1);
#pragma unroll  // (unrolled: the operand addresses of all 16 products are constants then, and this thread's instruction count bounds the kernel)
            for (int ch = 0; ch < 2; ++ch) {
              // P^T | dS^T arrive in two chunks: every compute warp's first 32 query columns (k-steps
              // 0, 1, 4, 5 of the 128 queries), then its other 32 (k-steps 2, 3, 6, 7)
              ok = settle(ch == 0 ? pr0 : pr1, &ctl->pds_ready[ch], g & 1);
              // the item's first products overwrite dK / dV: the previous item's must have been read out
              if (ok && it == 0 && ch == 0 && nk > 0) ok = mbar_wait<kMmaPollNs>(&ctl->acc_free, (nk - 1) & 1, err, kErrWaitMma);
              if (!ok) break;
              if (ch == 1 && has_dp) pr_do = mbar_try_wait(&ctl->do_full[sd], (tp >> 1) & 1);
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
            mma_commit(&ctl->do_free[g & 1]);         // (dP^T of this tile, the stage's other reader, was issued before)
            mma_commit(&ctl->q_free[g % kQStages]);   // (S^T of this tile, the stage's other reader, was issued before)
            if (it + 1 == n_iter) mma_commit(&ctl->done);
          }
          if (has_dp) {
            // dP^T of the next query tile (it overwrites P^T | dS^T of this one: ordered behind their readers above)
            ok = settle(pr_do, &ctl->do_full[sd], (tp >> 1) & 1);
            if (!ok) break;
            if (has_s) {
              pr_q = mbar_try_wait(&ctl->q_full[sq], (ts / kQStages) & 1);
              pr_sl = ts > 0 ? mbar_try_wait(&ctl->s_loaded, (ts - 1) & 1) : true;
            }
            tc_fence_after();
            const uint64_t dDOs = dDOk + sd * kTile16;
#pragma unroll
            for (int k = 0; k < 8; ++k) {
              const uint32_t off = ((k >> 2) * kBoxBytes + (k & 3) * 32) >> 4;
              mma_ss(tB, dV + off, dDOs + off, id_kk, k > 0 ? 1u : 0u);
            }
            mma_commit(&ctl->dp_ready);
            // that was the item's last read of V (its last read of K, S^T of the same tile, came earlier)
            if (it + 2 == n_iter) mma_commit(&ctl->kv_free);
          }
          if (has_s) {
            // S^T of the query tile after next, once the compute warps hold the tile before it in registers
            ok = settle(pr_q, &ctl->q_full[sq], (ts / kQStages) & 1);
            if (ok && ts > 0) ok = settle(pr_sl, &ctl->s_loaded, (ts - 1) & 1);
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
        gbase += n_iter;
        ++nk;
      }
    }
  } else {
    // -------------------------------------------------------------------- compute warps
    setmaxnreg_inc<208>();  // 128 x 80 + 256 x 208 <= 384 x 168 (the launch allocation)
    const int quad = warp & 3;
    const int half = (warp - 4) >> 2;            // which 64 query columns this warp handles
    const int row = quad * 32 + lane;            // key row
    const uint32_t lane_off = static_cast<uint32_t>(quad * 32) << 16;
    const float sl2 = p.scale_log2;
    bool ok = true;
    int gbase = 0, nk = 0;
    // An item's dK and dV are read out of tensor memory and stored only after the first exponentials
    // of the NEXT item: its last products are still running when its last dS^T has been handed over
    // (waiting for them right there left every compute warp idle), and the next item's first dV / dK
    // products are a whole tile's work away.  32 columns at a time through ONE copy of the code (a
    // thread owns 64 consecutive columns of one key row: 32-byte stores, whole sectors).
    bool pend = false;
    int pend_nk = 0, pend_sp = 0;
    long long pend_off = -1;  // element offset of this thread's 64 columns (-1: the key row does not exist)
    auto drain = [&]() -> bool {
      bool k = mbar_wait(&ctl->done, pend_nk & 1, err, kErrWaitEpilogue);
      k = __all_sync(0xffffffffu, k);
      if (!k) return false;
      tc_fence_after();
      const bool f32 = !kPlain && p.grad_fp32[pend_sp] != 0;
#pragma unroll 1
      for (int wc = 0; wc < 4; ++wc) {
        const int which = wc >> 1, c = wc & 1;
        uint32_t r[32];
        tmem_ld32((which == 0 ? tDK : tDV) + lane_off + half * 64 + c * 32, r);
        tmem_ld_wait();
        const float mul = which == 0 ? p.scale : 1.f;
        void* base = which == 0 ? p.dk[pend_sp] : p.dv[pend_sp];
        if (pend_off < 0) continue;
        if (f32) {
          float* dst = static_cast<float*>(base) + pend_off + c * 32;
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            uint32_t o[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) o[i] = __float_as_uint(__uint_as_float(r[v * 8 + i]) * mul);
            st_global_v8(dst + v * 8, o);
          }
        } else {
          uint16_t* dst = static_cast<uint16_t*>(base) + pend_off + c * 32;
#pragma unroll
          for (int v = 0; v < 2; ++v) {
            uint32_t o[8];
#pragma unroll
            for (int i = 0; i < 8; ++i)
              o[i] = pack2<kBf16>(__uint_as_float(r[v * 16 + 2 * i]) * mul, __uint_as_float(r[v * 16 + 2 * i + 1]) * mul);
            st_global_v8(dst + v * 16, o);
          }
        }
      }
      // every accumulator column of this warp has been read: the next item's products may overwrite them
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&ctl->acc_free);
      pend = false;
      return true;
    };

    for (int n = 0; ok; ++n) {
      const int slot = n & 1;
      ok = mbar_wait(&ctl->geom_full[slot], (n >> 1) & 1, err, kErrWaitSoftmax);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok || ctl->geom[slot].valid == 0) break;
      const BwdItemGeom gm = ctl->geom[slot];
      __syncwarp();
      if (lane == 0) mbar_arrive(&ctl->geom_free[slot]);
      const int n_iter = gm.n_qt * group;
      const bool valid_k = row < gm.n_valid_k;
      const int t = valid_k ? gm.t0 + row : 0x7fffffff;
      int p_hi = -1;
      if (valid_k) {
        int s_t, e_t;
        seq_of(cu_seq, n_seqs, t, s_t, e_t);
        const bool is_sink = t < s_t + n_sink;
        p_hi = (is_sink || e_t - 1 - t <= p.window) ? e_t - 1 : t + p.window;
        p_hi = min(p_hi, q_end_pos - 1);
      }

      int iq = 0;
      for (int it = 0; it < n_iter && ok; ++it) {
        const int g = gbase + it;
        const int pq0 = p.q_pos_start + (gm.qt_first + iq) * kTile;
        if (++iq == gm.n_qt) iq = 0;
        const float* lse_s = sLse + (g % kQStages) * kTile + half * 64;
        const float* del_s = sDelta + (g & 1) * kTile + half * 64;
        const bool full = (pq0 >= t) && (pq0 + kTile - 1 <= p_hi);
        const bool masked = !__all_sync(0xffffffffu, full);

        // P^T from S^T (the -lse2 row of this stage landed together with Q, before S^T was issued; the
        // rows arrive negated, see the delta kernel)
        ok = mbar_wait(&ctl->s_ready, g & 1, err, kErrWaitSoftmax);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        BWD_TRC(warp == 4 && lane == 0, g, 0);
        tc_fence_after();
        if (masked) {
          // A tile the band edge or a sequence boundary crosses gets its hidden scores replaced by -inf
          // IN tensor memory, by a short rolled loop, and then takes the same code as every other tile
          // (the compares unrolled over the 64 columns inside the loop below were a tenth of the
          // kernel, which has to fit the instruction cache).  This key sees the queries [t, p_hi].
          const uint32_t qn = static_cast<uint32_t>(max(p_hi - t + 1, 0));
#pragma unroll 1
          for (int c = 0; c < 2; ++c) {
            uint32_t sm[32];
            tmem_ld32(tS + lane_off + half * 64 + c * 32, sm);
            tmem_ld_wait();
            const int c0 = pq0 + half * 64 + c * 32 - t;
#pragma unroll
            for (int i = 0; i < 32; ++i) sm[i] = static_cast<uint32_t>(c0 + i) < qn ? sm[i] : 0xff800000u;
            tmem_st32(tS + lane_off + half * 64 + c * 32, sm);
          }
          tmem_st_wait();
        }
        float pr[64];
        {
          uint32_t s0[32], s1[32];
          tmem_ld32(tS + lane_off + half * 64, s0);
          tmem_ld32(tS + lane_off + half * 64 + 32, s1);
          tmem_ld_wait();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&ctl->s_loaded);  // S^T of the next query tile may overwrite these columns now
          // (two values per instruction wherever the pipe has a packed form)
          const float2 sl2v = make_float2(sl2, sl2);
#pragma unroll
          for (int i = 0; i < 32; i += 4) {
            const float4 la = *reinterpret_cast<const float4*>(lse_s + i);
            const float4 lb = *reinterpret_cast<const float4*>(lse_s + i + 32);
            const float2 xa01 = __ffma2_rn(make_float2(__uint_as_float(s0[i + 0]), __uint_as_float(s0[i + 1])), sl2v, make_float2(la.x, la.y));
            const float2 xa23 = __ffma2_rn(make_float2(__uint_as_float(s0[i + 2]), __uint_as_float(s0[i + 3])), sl2v, make_float2(la.z, la.w));
            const float2 xb01 = __ffma2_rn(make_float2(__uint_as_float(s1[i + 0]), __uint_as_float(s1[i + 1])), sl2v, make_float2(lb.x, lb.y));
            const float2 xb23 = __ffma2_rn(make_float2(__uint_as_float(s1[i + 2]), __uint_as_float(s1[i + 3])), sl2v, make_float2(lb.z, lb.w));
            // one pair in four goes through the FMA pipe instead of the special-function unit
            pr[i + 0] = ex2f(xa01.x), pr[i + 1] = ex2f(xa01.y);
            pr[i + 32] = ex2f(xb01.x), pr[i + 33] = ex2f(xb01.y);
            if (kBwdPoly && (i & 4)) {
              const float2 ea = ex2_poly2(xa23), eb = ex2_poly2(xb23);
              pr[i + 2] = ea.x, pr[i + 3] = ea.y, pr[i + 34] = eb.x, pr[i + 35] = eb.y;
            } else {
              pr[i + 2] = ex2f(xa23.x), pr[i + 3] = ex2f(xa23.y);
              pr[i + 34] = ex2f(xb23.x), pr[i + 35] = ex2f(xb23.y);
            }
          }
        }
        // Everything that does not need dP^T happens before the wait for it (the wait is on the loop
        // that bounds the kernel): P^T is packed, and -P^T * delta is formed so that one FMA per
        // element remains afterwards: dS^T = P^T * dP^T - P^T * delta.
        uint32_t ppk[32];
#pragma unroll
        for (int i = 0; i < 64; i += 2) ppk[i >> 1] = pack2<kBf16>(pr[i], pr[i + 1]);
        if (it == 0 && pend) {
          ok = drain();
          if (!ok) break;
        }
        // the delta row travels with the dO stage: it must have landed before it is read (the MMA
        // thread waits for the stage before dP^T, the compute warps have not waited for anything of it yet)
        ok = mbar_wait(&ctl->do_full[g & 1], (g >> 1) & 1, err, kErrWaitSoftmax);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        float npd[64];
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
          const float4 da = *reinterpret_cast<const float4*>(del_s + i);
          const float4 db = *reinterpret_cast<const float4*>(del_s + i + 32);
          const float2 n0 = __fmul2_rn(make_float2(pr[i + 0], pr[i + 1]), make_float2(da.x, da.y));
          const float2 n1 = __fmul2_rn(make_float2(pr[i + 2], pr[i + 3]), make_float2(da.z, da.w));
          const float2 n2 = __fmul2_rn(make_float2(pr[i + 32], pr[i + 33]), make_float2(db.x, db.y));
          const float2 n3 = __fmul2_rn(make_float2(pr[i + 34], pr[i + 35]), make_float2(db.z, db.w));
          npd[i + 0] = n0.x, npd[i + 1] = n0.y, npd[i + 2] = n1.x, npd[i + 3] = n1.y;
          npd[i + 32] = n2.x, npd[i + 33] = n2.y, npd[i + 34] = n3.x, npd[i + 35] = n3.y;
        }
        BWD_TRC(warp == 4 && lane == 0, g, 1);
        ok = mbar_wait(&ctl->dp_ready, g & 1, err, kErrWaitSoftmax);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        BWD_TRC(warp == 4 && lane == 0, g, 2);
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
              const float2 ds = __ffma2_rn(make_float2(pr[e], pr[e + 1]), make_float2(__uint_as_float(d[e]), __uint_as_float(d[e + 1])),
                                           make_float2(npd[e], npd[e + 1]));
              dd[i >> 1] = pack2<kBf16>(ds.x, ds.y);
            }
            tmem_st16(tB + lane_off + half * 64 + ch * 16, pp);
            tmem_st16(tB + lane_off + half * 64 + 32 + ch * 16, dd);
            tmem_st_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&ctl->pds_ready[ch]);
          }
        }
        BWD_TRC(warp == 4 && lane == 0, g, 3);
      }
      if (!ok) break;

      if (n_iter > 0) {
        // dK and dV of this key tile are read out and stored later, behind the first exponentials of the
        // next item (see drain above)
        pend = true;
        pend_nk = nk;
        pend_sp = gm.sp;
        pend_off = valid_k ? gm.b * p.dkv_sb[gm.sp] + static_cast<long long>(gm.key0 + row) * p.dkv_st[gm.sp] + gm.hk * p.dkv_sh[gm.sp] + half * 64 : -1;
        gbase += n_iter;
        ++nk;
      } else if (valid_k) {
        // no query of this call sees the tile: zero gradients
        const int sp = gm.sp;
        const long long off = gm.b * p.dkv_sb[sp] + static_cast<long long>(gm.key0 + row) * p.dkv_st[sp] + gm.hk * p.dkv_sh[sp] + half * 64;
        const bool f32 = !kPlain && p.grad_fp32[sp] != 0;
        const uint32_t z[8] = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u};
#pragma unroll 1
        for (int which = 0; which < 2; ++which) {
          void* base = which == 0 ? p.dk[sp] : p.dv[sp];
          const int n32 = f32 ? 8 : 4;  // 32-byte pieces of this thread's 64 columns
          uint8_t* dst = f32 ? reinterpret_cast<uint8_t*>(static_cast<float*>(base) + off) : reinterpret_cast<uint8_t*>(static_cast<uint16_t*>(base) + off);
#pragma unroll 1
          for (int v = 0; v < n32; ++v) st_global_v8(dst + v * 32, z);
        }
      }
      BWD_TRC(warp == 4 && lane == 0, gbase - 1, 5);
    }
    if (ok && pend) ok = drain();
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
  // one CTA per SM (shared memory and TMEM allow no more), each striding over the items
  const long long n_grid = n_cta < sm_count() ? n_cta : sm_count();
  kern<<<static_cast<unsigned>(n_grid), kBwdThreads, kBwdSmemBytes, stream>>>(kp, static_cast<int>(n_cta));
  e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_error("rswa_bwd: launch: %s", cudaGetErrorString(e));
    return RSWA_E_CUDA;
  }
  return RSWA_OK;
}

}  // namespace rswa
