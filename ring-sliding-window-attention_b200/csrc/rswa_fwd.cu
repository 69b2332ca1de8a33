// Forward kernel: banded (sliding-window + sink) softmax attention on the sm_100a tensor cores.
//
// One CTA owns two consecutive 128-row query tiles of one head and walks the key tiles either of
// them can see.  Two softmax warp groups (one per query tile) work in ping-pong against ONE
// MMA-issuing warp that serves the two query tiles strictly in turn, so that the tensor cores
// compute one tile's products while the other tile's exponentials run:
//
//   S_w = Q_w K^T      tcgen05.mma, both operands in shared memory (K-major), accumulator in TMEM
//   P_w = softmax      warp group w: one query row per thread, whole S row in registers, P written
//                      back (16-bit) over the same TMEM columns
//   O_w += P_w V       tcgen05.mma, A = P_w from TMEM, B = V from shared memory (MN-major)
//
// The issue order is  O_0 += P_0 V(j), S_0 = Q_0 K(j+1)^T, O_1 += P_1 V(j), S_1 = Q_1 K(j+1)^T, ...:
// S_w of the NEXT key tile goes right behind O_w += P_w V of the current one (tcgen05.mma
// instructions of one thread execute in issue order, so the overwrite of P_w's columns cannot
// overtake its last reader), and because everything comes from one thread the two tiles' products
// never interleave: S_0 becomes ready one product pair ahead of S_1, which keeps the two softmax
// groups half a period apart (with one issuing warp per tile the products of both tiles interleave
// on the tensor pipe, both S become ready together and the two groups run their exponentials at
// the same time, then both wait).  Loads travel in units of {K(j+1), V(j)}, the two tiles iteration
// j reads, through a two-stage ring.  The finished
// rows leave through shared memory so that every store instruction writes whole rows.
// TMEM: [0,128) S_0/P_0, [128,256) S_1/P_1, [256,384) O_0, [384,512) O_1.
//
// Key tiles that no row of the block can see are never loaded (rswa_tiles.cuh); a query tile skips
// the key tiles only the other one needs.  The math follows the reference's dense oracle
// (test/test_local_swa.py:51-93): scores scaled by softmax_scale, keys outside [p - W, p] masked
// (the sink columns forced on, test/test_local_slm.py:62-64), fp32 softmax, P rounded to the
// value dtype before P V.
#include "rswa_common.cuh"
#include "rswa_tiles.cuh"
#include "tc05.cuh"

namespace rswa {
using namespace tc05;

RSWA_TRACE_DECL(fwd)

namespace {

constexpr int kFwdThreads = 384;   // warp 0 TMA, warp 1 MMA, warps 2-3 idle, warps 4-7 / 8-11 softmax
constexpr int kFwdTmemCols = 512;
constexpr int kFwdSmemTiles = 7 * kTileBytes;  // Q_0, Q_1, K(0), 2 x {K(j+1), V(j)}
constexpr int kUnits = 2;

struct FwdCtl {
  uint64_t q_full, k0_full, kv_full[kUnits], kv_free[kUnits], s_ready[2], p_ready[2][2], pv_done[2];
  uint32_t tmem_base;
  int err;
  // which of the two query tiles need key tile j (bit w), written by the producer ahead of the load
  // that carries the tile's K and read by the MMA-issuing thread behind its wait for that load; two
  // units are in flight at most, so 8 slots are never overwritten while still unread
  uint32_t tile_flags[8];
  QBlockGeom geom;
};

constexpr int kFwdSmemBytes = kFwdSmemTiles + 1024;
static_assert(sizeof(FwdCtl) <= 1024, "control block too large");
static_assert(kFwdSmemBytes <= 232448, "shared memory budget");

// visible(p, t) for the row owning (lo, hi, seq, sink_end): t in [lo, hi] or a sink position <= hi
__device__ __forceinline__ bool key_visible(int t, int lo, int hi, int seq, int sink_end, int span_end) {
  return t <= hi && t < span_end && (t >= lo || (t >= seq && t < sink_end));
}

template <bool kBf16>
__global__ void __launch_bounds__(kFwdThreads, 1)
rswa_fwd_kernel(const __grid_constant__ FwdKernelParams p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* sQ = smem;                     // two query tiles
  uint8_t* sK0 = smem + 2 * kTileBytes;   // K of the first key tile
  uint8_t* sU = smem + 3 * kTileBytes;    // two units, each K(j+1) then V(j)
  FwdCtl* ctl = reinterpret_cast<FwdCtl*>(smem + kFwdSmemTiles);
  QBlockGeom* geom = &ctl->geom;

  RSWA_TRC(fwd, threadIdx.x == 0, 1920);
  // a device-side error was already reported on this stream: do not pile further time-outs on it
  if (__syncthreads_or(*reinterpret_cast<volatile int*>(p.status) != 0)) return;
  RSWA_TRC(fwd, threadIdx.x == 0, 1921);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // work item: query block fastest, then head, then batch row
  const int n_blocks = (p.n_q_tiles + 1) >> 1;
  int idx = blockIdx.x;
  const int blk = idx % n_blocks;
  idx /= n_blocks;
  const int h = idx % p.hq;
  const int b = idx / p.hq;
  const int hk = h / (p.hq / p.hkv);
  const int tile0 = p.q_tile_begin + 2 * blk;

  if (threadIdx.x == 0) {
    mbar_init(&ctl->q_full, 1);
    mbar_init(&ctl->k0_full, 1);
    for (int i = 0; i < kUnits; ++i) {
      mbar_init(&ctl->kv_full[i], 1);
      mbar_init(&ctl->kv_free[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&ctl->s_ready[i], 1);
      mbar_init(&ctl->p_ready[i][0], 4);  // one arrival per softmax warp and half of P
      mbar_init(&ctl->p_ready[i][1], 4);
      mbar_init(&ctl->pv_done[i], 1);
    }
    ctl->err = (smem_u32(smem) & 1023u) ? 199 : 0;
    mbar_fence_init();
    qblock_geometry<kTile>(geom, p.cu, p.n_seqs, p.n_spans, p.span_pos, p.span_len, p.q_pos_start, p.q_len,
                           p.window, p.n_sink, tile0, p.q_tile_begin + p.n_q_tiles);
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
  const int n_tiles = (ctl->err != 0) ? 0 : geom->n_tiles;
  RSWA_TRC(fwd, threadIdx.x == 0, 1922);

  if (warp < 4) {
    setmaxnreg_dec<88>();
    if (warp == 0 && lane == 0 && n_tiles > 0) {
      // ------------------------------------------------------------------ TMA producer
      // Loads travel in the order they are consumed: Q, K(0), then one unit per key tile j holding
      // K(j+1) and V(j) -- the two tiles iteration j of the MMA loop reads, so that one barrier fills
      // and one frees them.
      const bool two = geom->n_valid[1] > 0;
      mbar_expect_tx(&ctl->q_full, two ? 2 * kTileBytes : kTileBytes);
      tma_load_4d(sQ, &p.q_map, &ctl->q_full, 0, h, tile0 * kTile, b);
      tma_load_4d(sQ + kBoxBytes, &p.q_map, &ctl->q_full, 64, h, tile0 * kTile, b);
      if (two) {
        tma_load_4d(sQ + kTileBytes, &p.q_map, &ctl->q_full, 0, h, (tile0 + 1) * kTile, b);
        tma_load_4d(sQ + kTileBytes + kBoxBytes, &p.q_map, &ctl->q_full, 64, h, (tile0 + 1) * kTile, b);
      }
      TileCursor c, cn;
      cursor_begin<kTile>(geom, p.span_pos, p.span_len, c);
      ctl->tile_flags[0] = (tile_active(geom, 0, c, p.n_sink) ? 1u : 0u) | (tile_active(geom, 1, c, p.n_sink) ? 2u : 0u);
      mbar_expect_tx(&ctl->k0_full, kTileBytes);  // (release: the flags are visible to whoever sees the tile)
      tma_load_4d(sK0, &p.k_map[c.span], &ctl->k0_full, 0, hk, c.tok, b);
      tma_load_4d(sK0 + kBoxBytes, &p.k_map[c.span], &ctl->k0_full, 64, hk, c.tok, b);
      bool ok = true;
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int st = j & 1;
        const bool more = j + 1 < n_tiles;
        uint8_t* unit = sU + st * 2 * kTileBytes;
        cn = c;
        cursor_next<kTile>(geom, p.span_pos, p.span_len, cn, more);
        if (j >= kUnits) ok = mbar_wait<100>(&ctl->kv_free[st], ((j >> 1) - 1) & 1, err, kErrWaitProducer);
        if (!ok) break;
        RSWA_TRC(fwd, j < 32, j * 32 + 16);
        if (more)
          ctl->tile_flags[(j + 1) & 7] =
              (tile_active(geom, 0, cn, p.n_sink) ? 1u : 0u) | (tile_active(geom, 1, cn, p.n_sink) ? 2u : 0u);
        mbar_expect_tx(&ctl->kv_full[st], more ? 2 * kTileBytes : kTileBytes);
        if (more) {
          tma_load_4d(unit, &p.k_map[cn.span], &ctl->kv_full[st], 0, hk, cn.tok, b);
          tma_load_4d(unit + kBoxBytes, &p.k_map[cn.span], &ctl->kv_full[st], 64, hk, cn.tok, b);
        }
        tma_load_4d(unit + kTileBytes, &p.v_map[c.span], &ctl->kv_full[st], 0, hk, c.tok, b);
        tma_load_4d(unit + kTileBytes + kBoxBytes, &p.v_map[c.span], &ctl->kv_full[st], 64, hk, c.tok, b);
        c = cn;
      }
    } else if (warp == 1 && n_tiles > 0) {
      // ------------------------------------------------------------------ MMA issuer
      // ONE elected thread issues every product, the two query tiles strictly in turn, and does all the
      // waiting for them.  Its own instruction stream is the longest serial chain of the CTA (a lone
      // warp next to eight arithmetic-heavy ones gets an instruction through every 6-8 cycles), so it
      // does as little as possible: no geometry (which tiles matter to which query tile comes from the
      // producer's flags), one barrier per unit of loads, no warp votes.
      if (elect_one()) {
        constexpr uint32_t idesc_qk = idesc_f16(128, 128, kBf16 ? 1 : 0, 0, 0);
        constexpr uint32_t idesc_pv = idesc_f16(128, 128, kBf16 ? 1 : 0, 0, 1);
        // descriptors are built once; per stage / k-step only their address field moves (16-byte units)
        constexpr uint32_t kTile16 = kTileBytes >> 4;
        const uint64_t dQ = smem_desc_sw128(smem_u32(sQ), 16, 1024);
        const uint64_t dK0 = smem_desc_sw128(smem_u32(sK0), 16, 1024);
        const uint64_t dKu = smem_desc_sw128(smem_u32(sU), 16, 1024);
        const uint64_t dVu = smem_desc_sw128(smem_u32(sU) + kTileBytes, kBoxBytes, 1024);
        uint32_t pv_phase = 0;  // bit w: parity of p_ready[w][*] to wait for
        uint32_t pv_any = 0;    // bit w: O_w holds a product already (accumulate)
        bool ok = mbar_wait<0>(&ctl->q_full, 0, err, kErrWaitMma);
        if (ok) ok = mbar_wait<0>(&ctl->k0_full, 0, err, kErrWaitMma);
        uint32_t f_cur = 0;
        if (ok) {
          f_cur = ctl->tile_flags[0];
          tc_fence_after();
#pragma unroll
          for (int w = 0; w < 2; ++w) {
            if ((f_cur >> w) & 1u) {
#pragma unroll
              for (int k = 0; k < 8; ++k) {
                const uint32_t off = ((k >> 2) * kBoxBytes + (k & 3) * 32) >> 4;
                mma_ss(tmem + 128 * w, dQ + w * kTile16 + off, dK0 + off, idesc_qk, k > 0 ? 1u : 0u);
              }
              mma_commit(&ctl->s_ready[w]);
            }
          }
        }
        uint32_t kv_par = 0;  // parity of kv_full[j & 1] to wait for
        for (int j = 0; j < n_tiles && ok; ++j) {
          const bool more = j + 1 < n_tiles;
          const int st = j & 1;
          RSWA_TRC(fwd, j < 32, j * 32 + 24);
          ok = mbar_wait<0>(&ctl->kv_full[st], kv_par, err, kErrWaitMma);
          if (!ok) break;
          const uint32_t f_nxt = more ? ctl->tile_flags[(j + 1) & 7] : 0u;
          RSWA_TRC(fwd, j < 32, j * 32 + 0);
          const uint64_t dKs = dKu + st * (2 * kTile16);
          const uint64_t dVs = dVu + st * (2 * kTile16);
#pragma unroll
          for (int w = 0; w < 2; ++w) {
            const uint32_t tSw = tmem + 128 * w, tOw = tmem + 256 + 128 * w;
            if ((f_cur >> w) & 1u) {
#pragma unroll
              for (int half = 0; half < 2; ++half) {
                // P arrives in two halves of 64 keys: the first half of the product runs while the
                // second half's exponentials are still being computed
                ok = mbar_wait<0>(&ctl->p_ready[w][half], (pv_phase >> w) & 1u, err, kErrWaitMma);
                if (!ok) break;
                RSWA_TRC(fwd, j < 32, j * 32 + 1 + 4 * w + half);
                tc_fence_after();
#pragma unroll
                for (int k = 4 * half; k < 4 * half + 4; ++k) {
                  mma_ts(tOw, tSw + k * 8, dVs + k * 128, idesc_pv, (k > 0) ? 1u : ((pv_any >> w) & 1u));
                }
              }
              if (!ok) break;
              mma_commit(&ctl->pv_done[w]);
              RSWA_TRC(fwd, j < 32, j * 32 + 3 + 4 * w);
              pv_phase ^= 1u << w;
              pv_any |= 1u << w;
            }
            if ((f_nxt >> w) & 1u) {
              // overwrites P_w of the current tile: ordered behind the product just issued
#pragma unroll
              for (int k = 0; k < 8; ++k) {
                const uint32_t off = ((k >> 2) * kBoxBytes + (k & 3) * 32) >> 4;
                mma_ss(tSw, dQ + w * kTile16 + off, dKs + off, idesc_qk, k > 0 ? 1u : 0u);
              }
              mma_commit(&ctl->s_ready[w]);
              RSWA_TRC(fwd, j < 32, j * 32 + 4 + 4 * w);
            }
          }
          if (!ok) break;
          mma_commit(&ctl->kv_free[st]);
          f_cur = f_nxt;
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
    const bool valid = row < geom->n_valid[w];
    const int pos = geom->p0[w] + row;
    int s_p = 0, e_p = 0;
    if (valid) seq_of(p.cu, p.n_seqs, pos, s_p, e_p);
    // visible keys: [lo, hi] plus the sink positions [s_p, sink_end), all <= pos
    const int hi = valid ? pos : -1;
    const int lo = valid ? max(s_p, pos - p.window) : 0x7fffffff;
    const int sink_end = valid ? s_p + p.n_sink : -0x7fffffff;
    const float sl2 = p.scale_log2;

    float m_ref = -INFINITY;  // reference maximum in log2 units (already scaled)
    float l_sum = 0.f;
    int n_done = 0;           // key tiles this warp group has processed
    bool ok = true;
    TileCursor cur;
    cursor_begin<kTile>(geom, p.span_pos, p.span_len, cur);
    for (int j = 0; j < n_tiles && ok; ++j) {
      if (tile_active(geom, w, cur, p.n_sink)) {
        const int kt0 = cur.kt0;
        const int span_end = cur.kt_last + 1;
        ok = mbar_wait(&ctl->s_ready[w], n_done & 1, err, kErrWaitSoftmax);
        ok = __all_sync(0xffffffffu, ok);  // keep the warp converged for the TMEM accesses
        if (!ok) break;
        RSWA_TRC(fwd, lane == 0 && quad == 0 && j < 32, j * 32 + 10 + 8 * w);
        tc_fence_after();
        uint32_t r[128];
#pragma unroll
        for (int c = 0; c < 4; ++c) tmem_ld32(tS + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&r[c * 32]));
        tmem_ld_wait();
        RSWA_TRC(fwd, lane == 0 && quad == 0 && j < 32, j * 32 + 11 + 8 * w);
        // Mask.  Inside the tile this row sees the columns [c_lo, c_hi] (its window) and
        // [s_lo, s_hi) (sink tokens that lie below the window).  Almost every masked tile is either the
        // low edge of the band or the diagonal, where one compare per element is enough.
        const int c_lo = lo - kt0;
        const int c_hi = min(hi, span_end - 1) - kt0;
        const int s_lo = s_p - kt0;
        const int s_hi = min(min(sink_end, hi + 1), span_end) - kt0;
        const bool sink_here = s_lo < s_hi && s_hi > 0 && s_lo < kTile && s_lo < c_lo;
        if (__any_sync(0xffffffffu, sink_here)) {
#pragma unroll
          for (int i = 0; i < 128; ++i) {
            const bool vis = (i >= c_lo && i <= c_hi) || (i >= s_lo && i < s_hi);
            if (!vis) r[i] = 0xff800000u;  // -inf
          }
        } else {
          if (__any_sync(0xffffffffu, c_lo > 0)) {
#pragma unroll
            for (int i = 0; i < 128; ++i) r[i] = (i >= c_lo) ? r[i] : 0xff800000u;
          }
          if (__any_sync(0xffffffffu, c_hi < kTile - 1)) {
#pragma unroll
            for (int i = 0; i < 128; ++i) r[i] = (i <= c_hi) ? r[i] : 0xff800000u;
          }
        }
        float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
        for (int i = 0; i < 128; i += 8) {
          mx0 = fmax3(mx0, __uint_as_float(r[i]), __uint_as_float(r[i + 4]));
          mx1 = fmax3(mx1, __uint_as_float(r[i + 1]), __uint_as_float(r[i + 5]));
          mx2 = fmax3(mx2, __uint_as_float(r[i + 2]), __uint_as_float(r[i + 6]));
          mx3 = fmax3(mx3, __uint_as_float(r[i + 3]), __uint_as_float(r[i + 7]));
        }
        // Lazy rescale: keep the old reference maximum unless the new one exceeds it by more than
        // 2^8, so that O in TMEM is only touched rarely.
        const float mt = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * sl2;
        float alpha = 1.f;
        const bool grow = mt > m_ref + 8.f;
        if (grow) {
          alpha = ex2f(m_ref - mt);  // 0 when m_ref is -inf
          m_ref = mt;
        }
        if (n_done > 0 && __any_sync(0xffffffffu, grow)) {
          // O_w must be at rest: wait for the product of the previous tile
          ok = mbar_wait(&ctl->pv_done[w], (n_done - 1) & 1, err, kErrWaitSoftmax);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          tc_fence_after();
          l_sum *= alpha;
#pragma unroll 1
          for (int c = 0; c < 4; ++c) {
            uint32_t o[32];
            tmem_ld32(tO + c * 32, o);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st32(tO + c * 32, o);
          }
          tmem_st_wait();
        }
        RSWA_TRC(fwd, lane == 0 && quad == 0 && j < 32, j * 32 + 12 + 8 * w);
        const float m_use = (m_ref == -INFINITY) ? 0.f : m_ref;
        const float2 sl2v = make_float2(sl2, sl2), nmv = make_float2(-m_use, -m_use);
        float2 lacc = make_float2(0.f, 0.f);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t pk[16];
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const float2 x = __ffma2_rn(make_float2(__uint_as_float(r[c * 32 + i]), __uint_as_float(r[c * 32 + i + 1])),
                                        sl2v, nmv);
            const float2 e = make_float2(ex2f(x.x), ex2f(x.y));
            lacc = __fadd2_rn(lacc, e);
            pk[i >> 1] = pack2<kBf16>(e.x, e.y);
          }
          tmem_st16(tS + c * 16, pk);
          if (c & 1) {
            // a half of P (64 keys) is complete: its share of O_w += P_w V may start
            tmem_st_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&ctl->p_ready[w][c >> 1]);
            RSWA_TRC(fwd, lane == 0 && quad == 0 && j < 32, j * 32 + 13 + 8 * w + (c >> 1));
          }
        }
        l_sum += lacc.x + lacc.y;
        ++n_done;
      }
      cursor_next<kTile>(geom, p.span_pos, p.span_len, cur, j + 1 < n_tiles);
    }

    // epilogue: O / l -> out, lse
    RSWA_TRC(fwd, lane == 0 && quad == 0, 1924 + 4 * w);
    if (ok && n_done > 0) ok = mbar_wait(&ctl->pv_done[w], (n_done - 1) & 1, err, kErrWaitEpilogue);
    ok = __all_sync(0xffffffffu, ok);
    RSWA_TRC(fwd, lane == 0 && quad == 0, 1925 + 4 * w);
    tc_fence_after();
    const bool has = ok && n_done > 0 && l_sum > 0.f;
    const float inv = has ? 1.f / l_sum : 0.f;
    const int grow_q = (tile0 + w) * kTile + row;  // row inside the local q tensor
    if (n_done > 0 && ok) {
      // The rows go out through shared memory: a thread owns one 256-byte row, so storing from
      // registers would touch 32 different lines per instruction.  Staged in this warp's quarter of
      // the (no longer needed) Q tile, 16-byte chunks XOR-swizzled by row, each instruction then
      // writes two whole rows.  Only this warp touches the quarter: a warp-level sync suffices.
      uint8_t* stage = sQ + w * kTileBytes + quad * (32 * 256);
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t o[32];
        tmem_ld32(tO + c * 32, o);
        tmem_ld_wait();
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          uint4 q4;
          q4.x = pack2<kBf16>(__uint_as_float(o[v * 8 + 0]) * inv, __uint_as_float(o[v * 8 + 1]) * inv);
          q4.y = pack2<kBf16>(__uint_as_float(o[v * 8 + 2]) * inv, __uint_as_float(o[v * 8 + 3]) * inv);
          q4.z = pack2<kBf16>(__uint_as_float(o[v * 8 + 4]) * inv, __uint_as_float(o[v * 8 + 5]) * inv);
          q4.w = pack2<kBf16>(__uint_as_float(o[v * 8 + 6]) * inv, __uint_as_float(o[v * 8 + 7]) * inv);
          if (!has) q4 = make_uint4(0, 0, 0, 0);  // a row without a visible key
          *reinterpret_cast<uint4*>(stage + lane * 256 + (((c * 4 + v) ^ (lane & 15)) << 4)) = q4;
        }
      }
      __syncwarp();
      const int n_rows = geom->n_valid[w] - quad * 32;  // rows of this warp that exist
      uint16_t* obase = reinterpret_cast<uint16_t*>(p.out) + b * p.o_sb +
                        static_cast<long long>((tile0 + w) * kTile + quad * 32) * p.o_st + h * p.o_sh;
      const int ch = lane & 15;
#pragma unroll 4
      for (int i = 0; i < 16; ++i) {
        const int r = 2 * i + (lane >> 4);
        const uint4 q4 = *reinterpret_cast<const uint4*>(stage + r * 256 + ((ch ^ (r & 15)) << 4));
        if (r < n_rows) *reinterpret_cast<uint4*>(obase + static_cast<long long>(r) * p.o_st + ch * 8) = q4;
      }
    } else if (valid) {
      // no key of the given spans is visible to this query tile: zero rows
      uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(p.out) + b * p.o_sb +
                                            static_cast<long long>(grow_q) * p.o_st + h * p.o_sh);
#pragma unroll
      for (int v = 0; v < 16; ++v) dst[v] = make_uint4(0, 0, 0, 0);
    }
    if (valid) {
      p.lse[b * p.l_sb + h * p.l_sh + grow_q] = has ? (m_ref + log2f(l_sum)) * 0.6931471805599453f : -INFINITY;
    }
  }

  RSWA_TRC(fwd, lane == 0 && (warp == 4 || warp == 8), 1926 + (warp == 8 ? 4 : 0));
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
  const long long n_cta = static_cast<long long>((kp.n_q_tiles + 1) / 2) * kp.hq * kp.batch;
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
