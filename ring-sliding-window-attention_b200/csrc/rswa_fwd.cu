// Forward kernel: banded (sliding-window + sink) softmax attention on the sm_100a tensor cores.
//
// A work item is a block of two consecutive 128-row query tiles of one head; it walks the key tiles
// either of them can see.  Two softmax warp groups (one per query tile) work in ping-pong against
// ONE MMA-issuing thread that serves the two query tiles strictly in turn, so that the tensor cores
// compute one tile's products while the other tile's exponentials run:
//
//   S_w = Q_w K^T      tcgen05.mma, both operands in shared memory (K-major), accumulator in TMEM
//   P_w = softmax      warp group w: one query row per thread, whole S row in registers, P written
//                      back (16-bit) over the same TMEM columns, in two halves of 64 keys
//   O_w += P_w V       tcgen05.mma, A = P_w from TMEM, B = V from shared memory (MN-major)
//
// The issue order is  O_0 += P_0 V(g), S_0 = Q_0 K(g+1)^T, O_1 += P_1 V(g), S_1 = Q_1 K(g+1)^T, ...:
// S_w of the NEXT key tile goes right behind O_w += P_w V of the current one (tcgen05.mma
// instructions of one thread execute in issue order, so the overwrite of P_w's columns cannot
// overtake its last reader), and because everything comes from one thread the two tiles' products
// never interleave: S_0 becomes ready one product pair ahead of S_1, which keeps the two softmax
// groups half a period apart (with one issuing warp per tile the products of both tiles interleave
// on the tensor pipe, both S become ready together and the two groups run their exponentials at
// the same time, then both wait).
//
// The kernel is persistent: one CTA per SM strides over the items, and every pipeline keeps running
// across item boundaries.  Loads travel as a stream of units {K of the next key tile, V of the
// current one} -- the two tiles one step of the MMA loop reads -- through a two-stage ring; at an
// item boundary the unit simply carries the next item's first K tile, so S of the next item is
// computed while the softmax groups still normalise and store the rows of the finished one (staged
// through shared memory so that every store instruction writes whole row segments).
// TMEM: [0,128) S_0/P_0, [128,256) S_1/P_1, [256,384) O_0, [384,512) O_1.
//
// Key tiles that no row of the block can see are never loaded (rswa_tiles.cuh); a query tile skips
// the key tiles only the other one needs.  The math follows the reference's dense oracle
// (test/test_local_swa.py:51-93): scores scaled by softmax_scale, keys outside [p - W, p] masked
// (the sink columns forced on, test/test_local_slm.py:62-64), fp32 softmax, P rounded to the
// value dtype before P V.
#include "rswa_common.cuh"
#include "rswa_tiles.cuh"
#include <cuda_fp16.h>

#include "tc05.cuh"

namespace rswa {
using namespace tc05;

RSWA_TRACE_DECL(fwd)
#ifndef RSWA_TRACE_ITEM
#define RSWA_TRACE_ITEM 1
#define RSWA_TRACE_UNIT0 12
#endif

namespace {

constexpr int kFwdThreads = 384;   // warp 0 TMA, warp 1 MMA, warps 2-3 idle, warps 4-7 / 8-11 softmax
constexpr int kFwdTmemCols = 512;
constexpr int kFwdSmemTiles = 7 * kTileBytes;  // Q_0, Q_1, output staging (one tile), 2 units of {K, V}
constexpr int kUnits = 2;
constexpr int kSoftmaxWarps = 8;
#ifndef RSWA_FWD_POLY_EVERY
#define RSWA_FWD_POLY_EVERY 0
#endif
// n > 0: one pair of exponentials in n goes through a cubic on the FMA pipe instead of the special-function
// unit.  0 (every exponential on the special-function unit) measured fastest once the S row stayed in
// registers: 1.24 ms against 1.27 (n = 4), 1.28 (3), 1.31 (2) on the benchmark workload -- the softmax warps
// are bound by their instruction count, and the polynomial costs six times the instructions.
constexpr int kPolyEvery = RSWA_FWD_POLY_EVERY;

// flags of a unit, written by the producer ahead of the unit's loads
enum : uint32_t {
  kActMask = 3u,     // bit w: the unit's K tile matters to query tile w
  kFirst = 4u,       // the K tile is the first of its item (the products use a new Q, O starts over)
  kLast = 8u,        // ... the last of its item (Q may be replaced once its S products are done)
  kHasK = 16u,       // the unit carries a K tile
  kHasV = 32u,       // the unit carries the V tile of the previous unit's K tile
  kStop = 64u,       // nothing follows
};

struct FwdCtl {
  uint64_t q_full, q_free, kv_full[kUnits], kv_free[kUnits];
  uint64_t s_ready[2], p_ready[2][2], pv_done[2], o_free[2];
  uint64_t geom_full[2], geom_free[2];
  uint32_t tmem_base;
  int err;
  // two units are in flight at most, so 8 slots are never overwritten while still unread
  uint32_t unit_flags[8];
  int item[2];  // work item of each geometry slot, -1: no more work
  QBlockGeom geom[2];
};

constexpr int kFwdSmemBytes = kFwdSmemTiles + 1024;
static_assert(sizeof(FwdCtl) <= 1024, "control block too large");
static_assert(kFwdSmemBytes <= 232448, "shared memory budget");

struct FwdItem {
  int blk, h, b, hk, tile0;
};
__device__ __forceinline__ FwdItem fwd_item(const FwdKernelParams& p, int n_blocks, int it) {
  FwdItem d;  // query block fastest (late blocks, which see the most keys, first), then head, then batch row
  d.blk = n_blocks - 1 - it % n_blocks;
  it /= n_blocks;
  d.h = it % p.hq;
  d.b = it / p.hq;
  d.hk = d.h / (p.hq / p.hkv);
  d.tile0 = p.q_tile_begin + 2 * d.blk;
  return d;
}

// The SM's instruction cache holds 32 KB (measured: straight-line code in a loop runs at one instruction
// per cycle up to 32 KB and at half that beyond, and every jump into code that has left the cache
// costs a round trip to L2).  The three roles of this kernel together execute more than that per
// work item, so whatever a call cannot need is compiled out of its variant:
// kCarry:  out / lse hold a partial result that the call continues;
// kSimple: one KV span, no packed sequences, no sink tokens (the plain sliding window of one GPU, and
//          the tiles of a ring call that need no halo): the geometry collapses to a few lines.
template <bool kBf16, bool kCarry, bool kSimple>
__global__ void __launch_bounds__(kFwdThreads, 1)
rswa_fwd_kernel(const __grid_constant__ FwdKernelParams p, int n_blocks, int n_items) {
  const int* const cu_seq = kSimple ? nullptr : p.cu;
  const int n_seqs = kSimple ? 0 : p.n_seqs;
  const int n_spans = kSimple ? 1 : p.n_spans;
  const int n_sink = kSimple ? 0 : p.n_sink;
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* sQ = smem;                       // two query tiles
  uint8_t* sStage = smem + 2 * kTileBytes;  // output staging: 16 KB per softmax group
  uint8_t* sU = smem + 3 * kTileBytes;      // two units, each a K tile then a V tile
  FwdCtl* ctl = reinterpret_cast<FwdCtl*>(smem + kFwdSmemTiles);

  RSWA_TRC(fwd, threadIdx.x == 0, 1920);
  // a device-side error was already reported on this stream: do not pile further time-outs on it
  if (__syncthreads_or(*reinterpret_cast<volatile int*>(p.status) != 0)) return;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    mbar_init(&ctl->q_full, 1);
    mbar_init(&ctl->q_free, 1);
    for (int i = 0; i < kUnits; ++i) {
      mbar_init(&ctl->kv_full[i], 1);
      mbar_init(&ctl->kv_free[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&ctl->s_ready[i], 1);
      mbar_init(&ctl->p_ready[i][0], 4);  // one arrival per softmax warp and half of P
      mbar_init(&ctl->p_ready[i][1], 4);
      mbar_init(&ctl->pv_done[i], 1);
      mbar_init(&ctl->o_free[i], 4);
      mbar_init(&ctl->geom_full[i], 1);
      mbar_init(&ctl->geom_free[i], kSoftmaxWarps);
    }
    ctl->err = (smem_u32(smem) & 1023u) ? 199 : 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(&ctl->tmem_base, kFwdTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();

  const uint32_t tmem = ctl->tmem_base;
  volatile int* err = &ctl->err;
  const int n_work = (ctl->err != 0) ? 0 : n_items;
  RSWA_TRC(fwd, threadIdx.x == 0, 1922);

  if (warp < 4) {
    setmaxnreg_dec<88>();
    if (warp == 0 && lane == 0) {
      // ------------------------------------------------------------------ geometry + TMA producer
      // Walks the items of this CTA, prepares each item's key-tile list one item ahead (two-slot
      // ring) and streams the units.  Unit u carries the K tile of step u and the V tile of step
      // u - 1; the V tile of an item's last key tile travels with the next item's first K tile, or
      // alone when the next item has no key tile (or does not exist).
      // One loop turn per unit and ONE copy of everything a unit needs (the wait for its stage, its
      // flags, its loads): the thread runs through cold code at the pace of instruction fetch.
      int u = 0, ic = 0;       // units issued, items with work so far
      int n = -1, j = 0, n_tiles = 0;  // item of this CTA, next key tile of it, its key tiles
      bool more = true;        // items may follow
      bool pend = false;       // a V tile still to be sent
      int pv_span = 0, pv_tok = 0, pv_hk = 0, pv_b = 0;
      FwdItem w = {};
      QBlockGeom* geom = nullptr;
      TileCursor c = {};
      for (;;) {
        if (more && j >= n_tiles) {  // next item
          ++n;
          const int slot = n & 1;
          if (n >= 2 && !mbar_wait<100>(&ctl->geom_free[slot], ((n >> 1) - 1) & 1, err, kErrWaitProducer)) break;
          const int it = static_cast<int>(blockIdx.x) + n * static_cast<int>(gridDim.x);
          j = 0;
          if (it >= n_work) {  // tell the softmax warps that the work has run out
            ctl->item[slot] = -1;
            n_tiles = 0;
            more = false;
          } else {
            w = fwd_item(p, n_blocks, it);
            geom = &ctl->geom[slot];
            qblock_geometry<kTile>(geom, cu_seq, n_seqs, n_spans, p.span_pos, p.span_len, p.q_pos_start, p.q_len,
                                   p.window, n_sink, w.tile0, p.q_tile_begin + p.n_q_tiles);
            ctl->item[slot] = it;
            n_tiles = geom->n_tiles;
            cursor_begin<kTile>(geom, p.span_pos, p.span_len, c);
          }
          mbar_arrive(&ctl->geom_full[slot]);
        }
        const bool has_k = j < n_tiles;
        // (an item without key tiles: the finished item's last V tile must not wait for an item that
        // may never come, it travels alone)
        if (!has_k && !pend && more) continue;
        uint32_t flags = kStop;
        if (has_k) {
          flags = (tile_active(geom, 0, c, n_sink) ? 1u : 0u) | (tile_active(geom, 1, c, n_sink) ? 2u : 0u) |
                  (j == 0 ? kFirst : 0u) | (j + 1 == n_tiles ? kLast : 0u) | kHasK | (pend ? kHasV : 0u);
        } else if (pend) {
          flags = kHasV;
        }
        const int st = u & 1;
        if (u >= kUnits && !mbar_wait<100>(&ctl->kv_free[st], ((u >> 1) - 1) & 1, err, kErrWaitProducer)) break;
        ctl->unit_flags[u & 7] = flags;
        const uint32_t bytes = (has_k ? kTileBytes : 0) + (pend ? kTileBytes : 0);
        if (bytes > 0) mbar_expect_tx(&ctl->kv_full[st], bytes);  // (release: the flags are visible to whoever sees the unit)
        else mbar_arrive(&ctl->kv_full[st]);
        uint8_t* dst = sU + st * 2 * kTileBytes;
        if (pend) {
          tma_load_4d(dst + kTileBytes, &p.v_map[pv_span], &ctl->kv_full[st], 0, pv_hk, pv_tok, pv_b);
          tma_load_4d(dst + kTileBytes + kBoxBytes, &p.v_map[pv_span], &ctl->kv_full[st], 64, pv_hk, pv_tok, pv_b);
        }
        ++u;
        if (!has_k) {
          if (!pend) break;  // that was the stop unit
          pend = false;
          continue;
        }
        RSWA_TRC(fwd, n == RSWA_TRACE_ITEM && j < 32, j * 32 + 16);
        tma_load_4d(dst, &p.k_map[c.span], &ctl->kv_full[st], 0, w.hk, c.tok, w.b);
        tma_load_4d(dst + kBoxBytes, &p.k_map[c.span], &ctl->kv_full[st], 64, w.hk, c.tok, w.b);
        pend = true;
        pv_span = c.span, pv_tok = c.tok, pv_hk = w.hk, pv_b = w.b;
        if (j == 0) {
          // Q of this item, once the last S product of the previous item has read the old one
          if (ic > 0 && !mbar_wait<100>(&ctl->q_free, (ic - 1) & 1, err, kErrWaitProducer)) break;
          ++ic;
          const int n_q = geom->n_valid[1] > 0 ? 2 : 1;
          mbar_expect_tx(&ctl->q_full, n_q * kTileBytes);
#pragma unroll 1
          for (int i = 0; i < 2 * n_q; ++i) {
            tma_load_4d(sQ + (i >> 1) * kTileBytes + (i & 1) * kBoxBytes, &p.q_map, &ctl->q_full, (i & 1) * 64, w.h,
                        (w.tile0 + (i >> 1)) * kTile, w.b);
          }
        }
        ++j;
        cursor_next<kTile>(geom, p.span_pos, p.span_len, c, j < n_tiles);
      }
    } else if (warp == 1) {
      // ------------------------------------------------------------------ MMA issuer
      // ONE elected thread issues every product, the two query tiles strictly in turn, and does all the
      // waiting for them.  Its own instruction stream is the longest serial chain of the CTA (a lone
      // warp next to eight arithmetic-heavy ones gets an instruction through every 6-8 cycles), so it
      // does as little as possible: no geometry (what a unit holds and which query tile it matters to
      // comes from the producer's flags), one barrier per unit of loads, no warp votes.
      if (elect_one() && n_work > 0) {
        constexpr uint32_t idesc_qk = idesc_f16(128, 128, kBf16 ? 1 : 0, 0, 0);
        constexpr uint32_t idesc_pv = idesc_f16(128, 128, kBf16 ? 1 : 0, 0, 1);
        // descriptors are built once; per stage / k-step only their address field moves (16-byte units)
        constexpr uint32_t kTile16 = kTileBytes >> 4;
        const uint64_t dQ = smem_desc_sw128(smem_u32(sQ), 16, 1024);
        const uint64_t dKu = smem_desc_sw128(smem_u32(sU), 16, 1024);
        const uint64_t dVu = smem_desc_sw128(smem_u32(sU) + kTileBytes, kBoxBytes, 1024);
        uint32_t pv_phase = 0;  // bit w: parity of p_ready[w][*] to wait for
        uint32_t pv_any = 0;    // bit w: O_w holds a product of the current item already (accumulate)
        uint32_t of_cnt0 = 0, of_cnt1 = 0;  // items that have used O_w so far (phase of o_free[w])
        uint32_t q_par = 0, kv_par = 0;
        uint32_t f_prev = 0;    // flags of the unit whose K tile awaits its P V products
        bool ok = true;
        for (int u = 0; ok; ++u) {
          const int st = u & 1;
          RSWA_TRC(fwd, u >= RSWA_TRACE_UNIT0 && u < RSWA_TRACE_UNIT0 + 32, (u - RSWA_TRACE_UNIT0) * 32 + 24);
          ok = mbar_wait<0>(&ctl->kv_full[st], kv_par, err, kErrWaitMma);
          if (!ok) break;
          const uint32_t f = ctl->unit_flags[u & 7];
          if (f & kStop) break;
          RSWA_TRC(fwd, u >= RSWA_TRACE_UNIT0 && u < RSWA_TRACE_UNIT0 + 32, (u - RSWA_TRACE_UNIT0) * 32 + 0);
          bool need_q = (f & kFirst) != 0;  // the S products below are the first to read a new Q
          tc_fence_after();
          const uint64_t dKs = dKu + st * (2 * kTile16);
          const uint64_t dVs = dVu + st * (2 * kTile16);
#pragma unroll 1  // (one copy of the code for both query tiles: the thread is paced by instruction fetch, not by its arithmetic)
          for (int w = 0; w < 2; ++w) {
            const uint32_t tSw = tmem + 128 * w, tOw = tmem + 256 + 128 * w;
            if ((f & kHasV) && ((f_prev >> w) & 1u)) {
              if (!((pv_any >> w) & 1u)) {
                // first product of an item into O_w: the previous item's rows must have been read out
                const uint32_t cnt = w == 0 ? of_cnt0 : of_cnt1;
                if (cnt > 0) ok = mbar_wait<0>(&ctl->o_free[w], (cnt - 1) & 1u, err, kErrWaitMma);
                if (!ok) break;
              }
#pragma unroll
              for (int half = 0; half < 2; ++half) {
                // P arrives in two halves of 64 keys: the first half of the product runs while the
                // second half's exponentials are still being computed
                ok = mbar_wait<0>(&ctl->p_ready[w][half], (pv_phase >> w) & 1u, err, kErrWaitMma);
                if (!ok) break;
                RSWA_TRC(fwd, u >= RSWA_TRACE_UNIT0 && u < RSWA_TRACE_UNIT0 + 32, (u - RSWA_TRACE_UNIT0) * 32 + 1 + 4 * w + half);
                tc_fence_after();
#pragma unroll
                for (int k = 4 * half; k < 4 * half + 4; ++k) {
                  mma_ts(tOw, tSw + k * 8, dVs + k * 128, idesc_pv, (k > 0 || kCarry) ? 1u : ((pv_any >> w) & 1u));
                }
              }
              if (!ok) break;
              mma_commit(&ctl->pv_done[w]);
              RSWA_TRC(fwd, u >= RSWA_TRACE_UNIT0 && u < RSWA_TRACE_UNIT0 + 32, (u - RSWA_TRACE_UNIT0) * 32 + 3 + 4 * w);
              pv_phase ^= 1u << w;
              pv_any |= 1u << w;
            }
            if ((f & kHasK) && ((f >> w) & 1u)) {
              if (need_q) {  // the new item's Q (its load was issued right behind this unit's)
                ok = mbar_wait<0>(&ctl->q_full, q_par, err, kErrWaitMma);
                if (!ok) break;
                tc_fence_after();
                q_par ^= 1u;
                need_q = false;
              }
              // overwrites P_w of the previous key tile: ordered behind the product just issued
#pragma unroll
              for (int k = 0; k < 8; ++k) {
                const uint32_t off = ((k >> 2) * kBoxBytes + (k & 3) * 32) >> 4;
                mma_ss(tSw, dQ + w * kTile16 + off, dKs + off, idesc_qk, k > 0 ? 1u : 0u);
              }
              mma_commit(&ctl->s_ready[w]);
              RSWA_TRC(fwd, u >= RSWA_TRACE_UNIT0 && u < RSWA_TRACE_UNIT0 + 32, (u - RSWA_TRACE_UNIT0) * 32 + 4 + 4 * w);
            }
          }
          if (!ok) break;
          mma_commit(&ctl->kv_free[st]);
          if (f & kLast) mma_commit(&ctl->q_free);  // that was the item's last read of Q
          if ((f_prev & kLast) && (f & kHasV)) {
            // the products above were the last of their item
            if (pv_any & 1u) ++of_cnt0;
            if (pv_any & 2u) ++of_cnt1;
            pv_any = 0;
          }
          f_prev = (f & kHasK) ? f : 0u;
          if (st) kv_par ^= 1u;
        }
      }
      __syncwarp();
    }
  } else {
    // -------------------------------------------------------------------- softmax warp groups
    setmaxnreg_inc<208>();  // 128 x 88 + 256 x 208 <= 384 x 168 (the launch allocation)
    const int w = (warp - 4) >> 2;          // query tile of the block this warp group owns
    const int quad = warp & 3;              // TMEM lane quadrant this warp may touch
    const int row = quad * 32 + lane;       // query row inside the tile
    const uint32_t lane_off = static_cast<uint32_t>(quad * 32) << 16;
    const uint32_t tS = tmem + 128 * w + lane_off;
    const uint32_t tO = tmem + 256 + 128 * w + lane_off;
    const float sl2 = p.scale_log2;
    uint8_t* stage = sStage + w * (kTileBytes / 2) + quad * 4096;  // this warp's 32 rows x 128 bytes
    int n_tot = 0;   // key tiles this warp group has processed so far, all items (barrier phases)
    bool ok = true;

    for (int n = 0; ok; ++n) {
      const int slot = n & 1;
      ok = mbar_wait(&ctl->geom_full[slot], (n >> 1) & 1, err, kErrWaitSoftmax);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      const int it = ctl->item[slot];
      if (it < 0) break;
      RSWA_TRC(fwd, lane == 0 && warp == 4 && n < 64, 1024 + n);
      const FwdItem wi = fwd_item(p, n_blocks, it);
      const QBlockGeom* geom = &ctl->geom[slot];
      const int n_tiles = geom->n_tiles;
      const bool valid = row < geom->n_valid[w];
      const int pos = geom->p0[w] + row;
      int s_p = 0, e_p = 0;
      // (rows past the end look their sequence up at the last row that exists, so that s_p grows with the row)
      seq_of(cu_seq, n_seqs, geom->p0[w] + min(row, max(geom->n_valid[w], 1) - 1), s_p, e_p);
      // visible keys: [lo, hi] plus the sink positions [s_p, sink_end), all <= pos; nothing for rows
      // that do not exist
      const int hi = valid ? pos : -1;
      const int lo = valid ? max(s_p, pos - p.window) : 0x7fffffff;
      const int sink_end = valid ? s_p + n_sink : -0x7fffffff;
      // warp-uniform bounds for choosing the mask path of each 32-column chunk without a vote (a warp
      // with rows that do not exist gets bounds that send every chunk down the per-element path)
      const int lo_min = __reduce_min_sync(0xffffffffu, lo), lo_max = __reduce_max_sync(0xffffffffu, lo);
      const int hi_min = __reduce_min_sync(0xffffffffu, hi), hi_max = __reduce_max_sync(0xffffffffu, hi);
      const int sp_first = __shfl_sync(0xffffffffu, s_p, 0);
      const int se_last = __shfl_sync(0xffffffffu, s_p, 31) + n_sink;

      float m_ref = -INFINITY;  // reference maximum in log2 units (already scaled)
      float l_sum = 0.f;
      int n_done = 0;           // key tiles of this item this warp group has processed
      TileCursor cur;
      cursor_begin<kTile>(geom, p.span_pos, p.span_len, cur);
      for (int j = 0; j < n_tiles && ok; ++j) {
        if (tile_active(geom, w, cur, n_sink)) {
          const int kt0 = cur.kt0;
          const int span_end = cur.kt_last + 1;
          if (kCarry && n_done == 0) {
            // Continue the partial result that out / lse already hold (over other keys): the running
            // maximum is its lse, its weight 1, and O starts as its rows (zero where it saw no key).
            // This warp read O of the previous item out before it got here, and the first product of
            // this item comes after the P this warp hands over further down.
            const long long orow = wi.b * p.o_sb + static_cast<long long>((wi.tile0 + w) * kTile + row) * p.o_st + wi.h * p.o_sh;
            const float lp = valid ? p.lse[wi.b * p.l_sb + wi.h * p.l_sh + (wi.tile0 + w) * kTile + row] : -INFINITY;
            const bool had = lp > -INFINITY;
            m_ref = had ? lp * 1.4426950408889634f : -INFINITY;
            l_sum = had ? 1.f : 0.f;
            const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(p.out) + orow);
#pragma unroll 1
            for (int c = 0; c < 4; ++c) {
              uint32_t o[32];
#pragma unroll
              for (int v4 = 0; v4 < 4; ++v4) {
                const uint4 x = had ? src[c * 4 + v4] : make_uint4(0, 0, 0, 0);
                const uint32_t xw[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  if constexpr (kBf16) {
                    o[v4 * 8 + 2 * e] = xw[e] << 16;
                    o[v4 * 8 + 2 * e + 1] = xw[e] & 0xffff0000u;
                  } else {
                    const __half2 hh = *reinterpret_cast<const __half2*>(&xw[e]);
                    const float2 ff = __half22float2(hh);
                    o[v4 * 8 + 2 * e] = __float_as_uint(ff.x);
                    o[v4 * 8 + 2 * e + 1] = __float_as_uint(ff.y);
                  }
                }
              }
              tmem_st32(tO + c * 32, o);
            }
            tmem_st_wait();
          }
          ok = mbar_wait(&ctl->s_ready[w], n_tot & 1, err, kErrWaitSoftmax);
          ok = __all_sync(0xffffffffu, ok);  // keep the warp converged for the TMEM accesses
          if (!ok) break;
          RSWA_TRC(fwd, lane == 0 && quad == 0 && n == RSWA_TRACE_ITEM && j < 32, j * 32 + 10 + 8 * w);
          tc_fence_after();
          // One hot path for every tile: the S row goes into registers in one round trip to tensor
          // memory and stays there for both passes, without a compare.  A tile the band edge, the
          // diagonal, a sequence boundary or a sink column crosses first gets its hidden scores
          // replaced by -inf IN tensor memory, by a short rolled loop over chunks of 32 columns (mask
          // code unrolled over the row inside the hot path made it several times longer, and the
          // kernel is paced by instruction fetch wherever the hot path outgrows the instruction cache).
          const bool sink_tile = n_sink > 0 && kt0 < se_last && kt0 + kTile > sp_first;
          const int top_all = min(hi_min, span_end - 1);
          if (sink_tile || kt0 < lo_max || kt0 + kTile - 1 > top_all) {
            // inside the tile this row sees the columns [c_lo, c_lo + wn) (its window) and, with sink
            // tokens below the window, [s_lo, s_lo + sn)
            const int c_lo = lo - kt0;
            const int c_hi = min(hi, span_end - 1) - kt0;
            const uint32_t wn = static_cast<uint32_t>(max(c_hi - c_lo + 1, 0));
            const int s_lo = s_p - kt0;
            const uint32_t sn = sink_tile ? static_cast<uint32_t>(max(min(min(sink_end, hi + 1), span_end) - kt0 - s_lo, 0)) : 0u;
#pragma unroll 1
            for (int c = 0; c < 4; ++c) {
              const int a = kt0 + 32 * c;
              if (!sink_tile && a >= lo_max && a + 31 <= top_all) continue;  // every row of the warp sees the whole chunk
              uint32_t r[32];
              tmem_ld32(tS + c * 32, r);
              tmem_ld_wait();
#pragma unroll
              for (int i = 0; i < 32; ++i) {
                const int col = c * 32 + i;
                const bool vis = static_cast<uint32_t>(col - c_lo) < wn || (!kSimple && static_cast<uint32_t>(col - s_lo) < sn);
                r[i] = vis ? r[i] : 0xff800000u;  // -inf
              }
              tmem_st32(tS + c * 32, r);
            }
            tmem_st_wait();
          }
          float2 lacc = make_float2(0.f, 0.f);
          uint32_t r[2][2][32];  // [half of the tile][chunk of 32 columns]
#pragma unroll
          for (int c = 0; c < 4; ++c) tmem_ld32(tS + c * 32, r[c >> 1][c & 1]);
          tmem_ld_wait();
          // pass 1: the row maximum
          auto max_chunk = [&](const uint32_t (&x)[32]) -> float {
            float m0 = fmax3(__uint_as_float(x[0]), __uint_as_float(x[1]), __uint_as_float(x[2]));
            float m1 = fmax3(__uint_as_float(x[3]), __uint_as_float(x[4]), __uint_as_float(x[5]));
#pragma unroll
            for (int i = 6; i < 30; i += 6) {
              m0 = fmax3(m0, __uint_as_float(x[i]), __uint_as_float(x[i + 1]));
              m1 = fmax3(m1, __uint_as_float(x[i + 3]), __uint_as_float(x[i + 4]));
              m0 = fmaxf(m0, __uint_as_float(x[i + 2]));
              m1 = fmaxf(m1, __uint_as_float(x[i + 5]));
            }
            return fmax3(m0, m1, fmaxf(__uint_as_float(x[30]), __uint_as_float(x[31])));
          };
          const float mx = fmaxf(fmaxf(max_chunk(r[0][0]), max_chunk(r[0][1])), fmaxf(max_chunk(r[1][0]), max_chunk(r[1][1])));
          RSWA_TRC(fwd, lane == 0 && quad == 0 && n == RSWA_TRACE_ITEM && j < 32, j * 32 + 11 + 8 * w);
          // Lazy rescale: keep the old reference maximum unless the new one exceeds it by more than 2^8,
          // so that O in TMEM is only touched rarely.
          const float mt = mx * sl2;
          float alpha = 1.f;
          const bool grow = mt > m_ref + 8.f;
          if (grow) {
            alpha = ex2f(m_ref - mt);  // 0 when m_ref is -inf
            m_ref = mt;
          }
          if ((n_done > 0 || kCarry) && __any_sync(0xffffffffu, grow)) {
            // O_w must be at rest: wait for the product of the previous tile (none yet on an item's first
            // tile, where O_w is the carried-in partial result this warp has just written)
            if (n_done > 0) {
              ok = mbar_wait(&ctl->pv_done[w], (n_tot - 1) & 1, err, kErrWaitSoftmax);
              ok = __all_sync(0xffffffffu, ok);
              if (!ok) break;
            }
            tc_fence_after();
            l_sum *= alpha;
#pragma unroll 1
            for (int c = 0; c < 8; ++c) {  // (in small pieces: the S row occupies most of the registers)
              uint32_t o[16];
              tmem_ld16(tO + c * 16, o);
              tmem_ld_wait();
#pragma unroll
              for (int i = 0; i < 16; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
              tmem_st16(tO + c * 16, o);
            }
            tmem_st_wait();
          }
          RSWA_TRC(fwd, lane == 0 && quad == 0 && n == RSWA_TRACE_ITEM && j < 32, j * 32 + 12 + 8 * w);
          const float m_use = (m_ref == -INFINITY) ? 0.f : m_ref;  // (a row that has seen no key yet)
          const float2 sl2v = make_float2(sl2, sl2), nmv = make_float2(-m_use, -m_use);
          // pass 2: exponentials.  The two halves of the tile go through ONE copy of the code (the second
          // half then moves into the first half's registers: 64 moves, against an instruction stream
          // twice as long).
#pragma unroll 1
          for (int half = 0; half < 2; ++half) {
#pragma unroll
            for (int c = 0; c < 2; ++c) {
              uint32_t pk[16];
#pragma unroll
              for (int i = 0; i < 32; i += 2) {
                const float2 x = __ffma2_rn(make_float2(__uint_as_float(r[0][c][i]), __uint_as_float(r[0][c][i + 1])), sl2v, nmv);
                // one pair in kPolyEvery goes through the FMA pipe instead of the special-function unit,
                // which would otherwise need as long for a tile's exponentials as the tensor cores for
                // its two products
                const float2 e = (kPolyEvery > 0 && ((i >> 1) % (kPolyEvery > 0 ? kPolyEvery : 1)) == (kPolyEvery - 1))
                                     ? ex2_poly2(x) : make_float2(ex2f(x.x), ex2f(x.y));
                lacc = __fadd2_rn(lacc, e);
                pk[i >> 1] = pack2<kBf16>(e.x, e.y);
              }
              // P (16-bit) goes over the first half of the S columns, all of which are in registers by now
              tmem_st16(tS + half * 32 + c * 16, pk);
            }
            // a half of P (64 keys) is complete: its share of O_w += P_w V may start
            tmem_st_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&ctl->p_ready[w][half]);
            RSWA_TRC(fwd, lane == 0 && quad == 0 && n == RSWA_TRACE_ITEM && j < 32, j * 32 + 13 + 8 * w + half);
#pragma unroll
            for (int c = 0; c < 2; ++c)
#pragma unroll
              for (int i = 0; i < 32; ++i) r[0][c][i] = r[1][c][i];
          }
          l_sum += lacc.x + lacc.y;
          ++n_done;
          ++n_tot;
        }
        cursor_next<kTile>(geom, p.span_pos, p.span_len, cur, j + 1 < n_tiles);
      }
      if (!ok) break;

      // epilogue: O / l -> out, lse
      RSWA_TRC(fwd, lane == 0 && quad == 0 && n == RSWA_TRACE_ITEM, 1924 + 4 * w);
      const int n_rows = geom->n_valid[w] - quad * 32;  // rows of this warp that exist
      const int tile_row0 = (wi.tile0 + w) * kTile;     // first row of the tile inside the local q tensor
      // (a row whose every score was masked keeps m_ref = -inf; the exponentials computed on the FMA pipe
      // leave l_sum a hair above zero for it, so the row sum is no test)
      const bool has = n_done > 0 && m_ref > -INFINITY && l_sum > 0.f;
      const float inv = has ? 1.f / l_sum : 0.f;
      if (n_done > 0) {
        ok = mbar_wait(&ctl->pv_done[w], (n_tot - 1) & 1, err, kErrWaitEpilogue);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        RSWA_TRC(fwd, lane == 0 && quad == 0 && n == RSWA_TRACE_ITEM, 1925 + 4 * w);
        tc_fence_after();
        uint32_t o[128];
#pragma unroll
        for (int c = 0; c < 4; ++c) tmem_ld32(tO + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&o[c * 32]));
        tmem_ld_wait();
        // the accumulator is in registers: the next item's first product may overwrite it
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&ctl->o_free[w]);
        // The rows go out through shared memory: a thread owns one 256-byte row, so storing from
        // registers would touch 32 different lines per instruction.  Staged in two passes of 128 bytes
        // per row (16-byte chunks XOR-swizzled by row), each store instruction then writes four
        // 128-byte row segments.  Only this warp touches its part of the staging buffer.
        uint16_t* obase = reinterpret_cast<uint16_t*>(p.out) + wi.b * p.o_sb +
                          static_cast<long long>(tile_row0 + quad * 32) * p.o_st + wi.h * p.o_sh;
        const int ch = lane & 7;
#pragma unroll 1  // (one copy of the code; the second half of the row moves down in the registers)
        for (int pass = 0; pass < 2; ++pass) {
#pragma unroll
          for (int v = 0; v < 8; ++v) {
            const int e0 = v * 8;
            uint4 q4;
            q4.x = pack2<kBf16>(__uint_as_float(o[e0 + 0]) * inv, __uint_as_float(o[e0 + 1]) * inv);
            q4.y = pack2<kBf16>(__uint_as_float(o[e0 + 2]) * inv, __uint_as_float(o[e0 + 3]) * inv);
            q4.z = pack2<kBf16>(__uint_as_float(o[e0 + 4]) * inv, __uint_as_float(o[e0 + 5]) * inv);
            q4.w = pack2<kBf16>(__uint_as_float(o[e0 + 6]) * inv, __uint_as_float(o[e0 + 7]) * inv);
            *reinterpret_cast<uint4*>(stage + lane * 128 + ((v ^ (lane & 7)) << 4)) = q4;
          }
          __syncwarp();
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int rr = 4 * i + (lane >> 3);
            const uint4 q4 = *reinterpret_cast<const uint4*>(stage + rr * 128 + ((ch ^ (rr & 7)) << 4));
            if (rr < n_rows) *reinterpret_cast<uint4*>(obase + static_cast<long long>(rr) * p.o_st + pass * 64 + ch * 8) = q4;
          }
          __syncwarp();  // the staging rows are rewritten by the next pass / item
#pragma unroll
          for (int i = 0; i < 64; ++i) o[i] = o[64 + i];
        }
      } else if (valid && !kCarry) {
        // no key of the given spans is visible to this query tile: zero rows (a carried-in partial
        // result stays as it is)
        uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(p.out) + wi.b * p.o_sb +
                                              static_cast<long long>(tile_row0 + row) * p.o_st + wi.h * p.o_sh);
#pragma unroll
        for (int v = 0; v < 16; ++v) dst[v] = make_uint4(0, 0, 0, 0);
      }
      if (valid && (n_done > 0 || !kCarry)) {
        p.lse[wi.b * p.l_sb + wi.h * p.l_sh + tile_row0 + row] =
            has ? (m_ref + log2f(l_sum)) * 0.6931471805599453f : -INFINITY;
      }
      RSWA_TRC(fwd, lane == 0 && quad == 0 && n == RSWA_TRACE_ITEM, 1926 + 4 * w);
      RSWA_TRC(fwd, lane == 0 && warp == 4 && n < 64, 1100 + n);
      __syncwarp();
      if (lane == 0) mbar_arrive(&ctl->geom_free[slot]);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, kFwdTmemCols);
  }
  RSWA_TRC(fwd, threadIdx.x == 32, 1923);
  if (threadIdx.x == 0 && ctl->err != 0) atomicCAS(p.status, 0, ctl->err);
}

}  // namespace

int launch_fwd(const FwdKernelParams& kp, int dtype, cudaStream_t stream) {
  const int n_blocks = (kp.n_q_tiles + 1) / 2;
  const long long n_items = static_cast<long long>(n_blocks) * kp.hq * kp.batch;
  if (n_items <= 0) return RSWA_OK;
  if (n_items > 0x7fffffffLL) {
    set_error("rswa_fwd: too many query tiles (%lld)", n_items);
    return RSWA_E_ARG;
  }
  const bool simple = kp.n_spans == 1 && kp.cu == nullptr && kp.n_sink == 0;
  const int variant = (dtype == RSWA_DTYPE_BF16 ? 1 : 0) + (kp.carry ? 2 : 0) + (simple ? 4 : 0);
  using Kern = void (*)(const FwdKernelParams, int, int);
  static const Kern kerns[8] = {rswa_fwd_kernel<false, false, false>, rswa_fwd_kernel<true, false, false>,
                                rswa_fwd_kernel<false, true, false>,  rswa_fwd_kernel<true, true, false>,
                                rswa_fwd_kernel<false, false, true>,  rswa_fwd_kernel<true, false, true>,
                                rswa_fwd_kernel<false, true, true>,   rswa_fwd_kernel<true, true, true>};
  const Kern kern = kerns[variant];
  // (the attribute is a property of the function on a device: set once per kernel variant and device)
  static bool attr_set[8][64] = {{false}};
  int dev_id = 0;
  cudaError_t e = cudaGetDevice(&dev_id);
  if (e == cudaSuccess && (dev_id < 0 || dev_id >= 64 || !attr_set[variant][dev_id])) {
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kFwdSmemBytes);
    if (e == cudaSuccess && dev_id >= 0 && dev_id < 64) attr_set[variant][dev_id] = true;
  }
  if (e != cudaSuccess) {
    set_error("rswa_fwd: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    return RSWA_E_CUDA;
  }
  // one CTA per SM (shared memory and TMEM allow no more), each striding over the items
  const long long n_cta = n_items < sm_count() ? n_items : sm_count();
  kern<<<static_cast<unsigned>(n_cta), kFwdThreads, kFwdSmemBytes, stream>>>(kp, n_blocks, static_cast<int>(n_items));
  e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_error("rswa_fwd: launch: %s", cudaGetErrorString(e));
    return RSWA_E_CUDA;
  }
  return RSWA_OK;
}

}  // namespace rswa
