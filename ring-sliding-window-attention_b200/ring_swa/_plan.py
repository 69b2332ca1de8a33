"""Host-side plan of one rank's halo and sink exchange.  Pure integer logic, no tensors.

The reference forwards WHOLE K/V blocks hop by hop round the ring for
C = min(ceil(W / S), cp - 1) rounds (ring_swa/sliding_window/nonvarlen.py:46-49, 70-92) and lets
each hop's mask case discard what is not visible.  Here every rank works out, from the same
inputs, exactly which trailing tokens of which earlier rank it can see, and only those travel:
rank r needs the keys at global positions [max(seq_start, r*S - W), r*S), i.e. the trailing
min(S, ...) tokens of ranks r-1, r-2, ..., plus (StreamingLLM) the first n_sink tokens of the
sequence that crosses its left edge, sent by the rank that owns them
(ring_swa/streaming_llm/nonvarlen.py:48-55 broadcasts them from group rank 0).

Chunks need not be equal: the reference assumes the same number of tokens on every rank
(ring_swa/sliding_window/varlen.py:56-59, its FIXME); with `chunk_lens` (one length per group rank)
rank r owns the positions [bounds[r], bounds[r+1]) of the packed token axis, bounds being the
running sum, and everything below works on those bounds.
"""
from __future__ import annotations

import bisect
from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Tuple

TILE = 128


@dataclass
class HaloRecv:
    hop: int          # source is group rank `rank - hop`
    src: int
    length: int       # trailing tokens of the source's chunk
    pos_start: int    # global position of the first of them


@dataclass
class HaloSend:
    hop: int
    dst: int
    length: int       # my trailing tokens


@dataclass
class SinkRecv:
    """One piece of the sink tokens: the part of them that one earlier rank holds.  The first n_sink
    tokens of a sequence that starts fewer than n_sink tokens before a chunk boundary (or n_sink > S)
    lie on several ranks, hence a list of pieces, one message each."""
    owner: int        # group rank that holds these sink tokens
    pos_start: int    # their global position
    n: int


@dataclass
class SinkSend:
    dst: int
    offset: int       # local token offset of the sink tokens in my chunk
    n: int


@dataclass
class RingPlan:
    cp: int
    rank: int
    seq_per_rank: int         # tokens on THIS rank
    window: int
    n_sink: int
    pos_start: int = 0        # global position of this rank's first token
    halo_recv: List[HaloRecv] = field(default_factory=list)
    halo_send: List[HaloSend] = field(default_factory=list)
    sink_recv: List[SinkRecv] = field(default_factory=list)   # ascending position, one per owning rank
    sink_send: List[SinkSend] = field(default_factory=list)
    # query tiles [halo_tile_end, n_tiles) see local keys only (and the sink)
    halo_tile_end: int = 0

    @property
    def q_pos_start(self) -> int:
        return self.pos_start

    @property
    def n_tiles(self) -> int:
        return (self.seq_per_rank + TILE - 1) // TILE


def seq_start_of(pos: int, cu: Optional[Sequence[int]]) -> int:
    """Start of the sequence that contains global position `pos` (0 when batch rows are the sequences)."""
    if cu is None:
        return 0
    i = bisect.bisect_right(cu, pos) - 1
    i = max(0, min(i, len(cu) - 2))
    return int(cu[i])


def chunk_bounds(cp: int, S: int, chunk_lens: Optional[Sequence[int]]) -> List[int]:
    """Global position of every rank's first token, plus the total: cp + 1 ascending numbers."""
    if chunk_lens is None:
        return [r * S for r in range(cp + 1)]
    lens = [int(x) for x in chunk_lens]
    if len(lens) != cp or any(x <= 0 for x in lens):
        raise ValueError(f"chunk lengths must be {cp} positive numbers, one per rank of the group: {lens}")
    bounds = [0]
    for x in lens:
        bounds.append(bounds[-1] + x)
    return bounds


def _needs(r: int, bounds: Sequence[int], W: int, n_sink: int, cu) -> Tuple[int, List[HaloRecv], List[SinkRecv]]:
    """What rank r must receive: (lowest needed window position, halos, sink).

    The sink tokens of the sequence that crosses the rank's left edge always travel as their own
    small message when they live on an earlier rank, even if the window reaches them: every query
    of that sequence needs them, also the ones that otherwise see local keys only and run before
    the halo has arrived.  The halo then starts behind the sink tokens, so the two never overlap.
    """
    left = bounds[r]
    s_cross = seq_start_of(left, cu)
    lo = max(s_cross, left - W, 0)
    sink: List[SinkRecv] = []
    if n_sink > 0 and s_cross < left:
        end = min(s_cross + n_sink, left)
        a = s_cross
        while a < end:  # one piece per rank that owns some of [s_cross, end)
            owner = bisect.bisect_right(bounds, a) - 1
            b = min(end, bounds[owner + 1])
            sink.append(SinkRecv(owner=owner, pos_start=a, n=b - a))
            a = b
        lo = max(lo, end)
    halos: List[HaloRecv] = []
    h = 1
    while r - h >= 0:
        a, b = bounds[r - h], bounds[r - h + 1]
        if b <= lo:
            break
        start = max(lo, a)
        halos.append(HaloRecv(hop=h, src=r - h, length=b - start, pos_start=start))
        h += 1
    return lo, halos, sink


def make_plan(cp: int, rank: int, S: int, W: int, n_sink: int, cu: Optional[Sequence[int]],
              chunk_lens: Optional[Sequence[int]] = None) -> RingPlan:
    """Plan for `rank`; every rank derives the matching sends from the other ranks' needs.
    `S` is the number of tokens on this rank; `chunk_lens` (all ranks' lengths) when they differ."""
    if cp < 1 or not (0 <= rank < cp):
        raise ValueError(f"invalid context-parallel geometry: cp_size={cp}, cp_local_rank={rank}")
    if S <= 0 or W < 0 or n_sink < 0:
        raise ValueError("sequence length per rank must be positive, window and n_sink non-negative")
    bounds = chunk_bounds(cp, S, chunk_lens)
    if bounds[rank + 1] - bounds[rank] != S:
        raise ValueError(f"rank {rank} holds {S} tokens but its chunk length is given as {bounds[rank + 1] - bounds[rank]}")
    plan = RingPlan(cp=cp, rank=rank, seq_per_rank=S, window=W, n_sink=n_sink, pos_start=bounds[rank])
    lo, plan.halo_recv, plan.sink_recv = _needs(rank, bounds, W, n_sink, cu)
    for r in range(rank + 1, cp):
        _, halos, sink = _needs(r, bounds, W, n_sink, cu)
        for hr in halos:
            if hr.src == rank:
                plan.halo_send.append(HaloSend(hop=hr.hop, dst=r, length=hr.length))
        for piece in sink:
            if piece.owner == rank:
                plan.sink_send.append(SinkSend(dst=r, offset=piece.pos_start - bounds[rank], n=piece.n))
    if plan.halo_recv:
        # local query a (position rank*S + a) reaches below the chunk iff a < W
        plan.halo_tile_end = min(plan.n_tiles, (min(W, S) + TILE - 1) // TILE)
    return plan
