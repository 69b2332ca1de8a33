// Key-tile enumeration shared by the query-stationary kernels (forward and dQ).
//
// A CTA owns a block of two consecutive 128-row query tiles of one head.  The keys any row of the
// block can see are one contiguous run of global positions [min_lo, max_hi] (plus the sink tokens
// of the sequence the block starts in), intersected with every KV span.  That intersection is
// stored as a short list of (span, first tile, tile count) entries; every role of the CTA walks
// the same list in the same order.  Whether a given key tile matters to query tile w of the block
// is a pure function of the tile's positions (tile_active), so all roles agree without talking.
#pragma once
#include "rswa_common.cuh"

namespace rswa {

struct QBlockGeom {
  int n_entries;
  int n_tiles;
  int ent_span[kMaxEntries];
  int ent_first[kMaxEntries];
  int ent_count[kMaxEntries];
  // per query tile of the block
  int n_valid[2];  // rows that exist (0: the tile is not part of this launch)
  int p0[2];       // global position of row 0
  int lo[2];       // lowest window position any row can see
  int hi[2];       // highest position (the last valid row's own)
  int seq0[2];     // start of the sequence row 0 lies in
};

// Filled by one thread.  kBN = key rows per tile (128 forward, 64 dQ).
template <int kBN>
__device__ inline void qblock_geometry(QBlockGeom* g, const int* cu, int n_seqs, int n_spans, const int* span_pos,
                                       const int* span_len, int q_pos_start, int q_len, int window, int n_sink,
                                       int tile0, int tile_end) {
  for (int w = 0; w < 2; ++w) {
    const int tile = tile0 + w;
    const int row0 = tile * kTile;
    int nv = (tile < tile_end) ? min(kTile, q_len - row0) : 0;
    nv = max(nv, 0);
    g->n_valid[w] = nv;
    g->p0[w] = q_pos_start + row0;
    int s = 0, e = 0;
    if (nv > 0) seq_of(cu, n_seqs, g->p0[w], s, e);
    g->seq0[w] = s;
    g->lo[w] = max(s, g->p0[w] - window);
    g->hi[w] = g->p0[w] + nv - 1;
  }
  int ne = 0, nt = 0;
  if (g->n_valid[0] > 0) {
    const int min_lo = g->lo[0];
    const int max_hi = g->n_valid[1] > 0 ? g->hi[1] : g->hi[0];
    const int s0 = g->seq0[0];
    for (int i = 0; i < n_spans; ++i) {
      const int a = span_pos[i], bnd = a + span_len[i];
      int wfirst = -1, wlast = -1;
      const int wl = max(min_lo, a), wh = min(max_hi, bnd - 1);
      if (wl <= wh) {
        wfirst = (wl - a) / kBN;
        wlast = (wh - a) / kBN;
      }
      if (n_sink > 0) {  // sink tiles that lie below the window tiles of this span
        const int sl = max(s0, a), sh = min(min(s0 + n_sink - 1, bnd - 1), max_hi);
        if (sl <= sh) {
          const int sf = (sl - a) / kBN;
          int slast = (sh - a) / kBN;
          if (wfirst >= 0) slast = min(slast, wfirst - 1);
          if (sf <= slast) {
            g->ent_span[ne] = i;
            g->ent_first[ne] = sf;
            g->ent_count[ne] = slast - sf + 1;
            nt += slast - sf + 1;
            ++ne;
          }
        }
      }
      if (wfirst >= 0) {
        g->ent_span[ne] = i;
        g->ent_first[ne] = wfirst;
        g->ent_count[ne] = wlast - wfirst + 1;
        nt += wlast - wfirst + 1;
        ++ne;
      }
    }
  }
  g->n_entries = ne;
  g->n_tiles = nt;
}

// Cursor over the tile list.
struct TileCursor {
  int e, t;      // entry, tile inside the entry
  int span;      // KV span of the current tile
  int tok;       // token offset of the tile inside the span
  int kt0;       // global position of its first key
  int kt_last;   // global position of its last existing key
};

template <int kBN>
__device__ __forceinline__ void cursor_load(const QBlockGeom* g, const int* span_pos, const int* span_len,
                                            TileCursor& c) {
  c.span = g->ent_span[c.e];
  c.tok = (g->ent_first[c.e] + c.t) * kBN;
  c.kt0 = span_pos[c.span] + c.tok;
  c.kt_last = min(c.kt0 + kBN - 1, span_pos[c.span] + span_len[c.span] - 1);
}
template <int kBN>
__device__ __forceinline__ void cursor_begin(const QBlockGeom* g, const int* span_pos, const int* span_len,
                                             TileCursor& c) {
  c.e = 0;
  c.t = 0;
  if (g->n_tiles > 0) cursor_load<kBN>(g, span_pos, span_len, c);
}
// Advances; the caller knows from its own count when the list is exhausted.
template <int kBN>
__device__ __forceinline__ void cursor_next(const QBlockGeom* g, const int* span_pos, const int* span_len,
                                            TileCursor& c, bool more) {
  if (!more) return;
  if (++c.t >= g->ent_count[c.e]) {
    c.t = 0;
    ++c.e;
  }
  cursor_load<kBN>(g, span_pos, span_len, c);
}

// Does any row of query tile w see a key of the tile under the cursor?
__device__ __forceinline__ bool tile_active(const QBlockGeom* g, int w, const TileCursor& c, int n_sink) {
  if (g->n_valid[w] <= 0 || c.kt0 > g->hi[w]) return false;
  if (c.kt_last >= g->lo[w]) return true;
  return n_sink > 0 && c.kt0 < g->seq0[w] + n_sink && c.kt_last >= g->seq0[w];
}

}  // namespace rswa
