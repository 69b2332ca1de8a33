"""Halo / sink plan: pure host logic."""
import math

import pytest

from ring_swa._plan import make_plan


@pytest.mark.parametrize("cp,S,W", [(8, 4096, 1000), (8, 32768, 65536), (4, 16, 5), (4, 16, 16), (4, 16, 17),
                                     (4, 16, 100), (2, 300, 0), (8, 512, 8000)])
def test_nonvarlen_halo_matches_reference_round_count(cp, S, W):
    # ring rounds of the reference: C = min(ceil(W / S), cp - 1), docs/implementation_details.md:17-21
    C = min(math.ceil(W / S), cp - 1)
    for r in range(cp):
        p = make_plan(cp, r, S, W, 0, None)
        assert len(p.halo_recv) == min(C, r)
        total = sum(h.length for h in p.halo_recv)
        assert total == min(W, r * S)
        # contiguous, ending at the rank's left edge
        pos = r * S
        for h in p.halo_recv:
            assert h.pos_start + h.length == pos and h.src == r - h.hop
            pos = h.pos_start
        assert not p.sink_recv and not p.sink_send


def test_sends_mirror_receives():
    for cu in (None, [0, 7, 8, 9, 40, 64], [0, 64], [0, 16, 32, 48, 64]):
        for W in (1, 5, 16, 17, 40, 100):
            for ns in (0, 1, 3):
                plans = [make_plan(4, r, 16, W, ns, cu) for r in range(4)]
                for r, p in enumerate(plans):
                    for h in p.halo_recv:
                        assert any(s.dst == r and s.length == h.length for s in plans[h.src].halo_send)
                    for piece in p.sink_recv:
                        o = piece.owner
                        assert any(s.dst == r and s.n == piece.n and
                                   s.offset + o * 16 == piece.pos_start for s in plans[o].sink_send)
                    n_recv = sum(1 for q in plans for h in q.halo_recv if h.src == r)
                    assert n_recv == len(p.halo_send)


def test_varlen_halo_stops_at_sequence_start():
    cu = [0, 30, 64]
    p = make_plan(4, 2, 16, 100, 0, cu)      # rank 2 starts at 32, its sequence at 30
    assert [(h.src, h.length, h.pos_start) for h in p.halo_recv] == [(1, 2, 30)]
    p = make_plan(4, 2, 16, 100, 0, [0, 32, 64])   # sequence starts exactly on the rank edge
    assert p.halo_recv == [] and p.halo_tile_end == 0


def test_sink_travels_separately_and_never_overlaps_the_halo():
    def only(plan):
        assert len(plan.sink_recv) == 1
        return plan.sink_recv[0]
    p = make_plan(4, 3, 16, 5, 1, None)
    assert (only(p).owner, only(p).pos_start, only(p).n) == (0, 0, 1)
    # window reaches token 0: the sink still has its own message and the halo starts behind it
    p = make_plan(4, 1, 16, 20, 1, None)
    assert (only(p).pos_start, only(p).n) == (0, 1)
    assert [(h.pos_start, h.length) for h in p.halo_recv] == [(1, 15)]
    p = make_plan(4, 1, 16, 14, 4, None)
    assert (only(p).pos_start, only(p).n) == (0, 4)
    assert [(h.pos_start, h.length) for h in p.halo_recv] == [(4, 12)]
    # the sequence starts on this rank: its sink is local, nothing extra travels
    assert make_plan(4, 2, 16, 5, 1, [0, 32, 64]).sink_recv == []
    assert make_plan(4, 0, 16, 5, 1, None).sink_recv == []
    # packed: the crossing sequence starts inside the window's reach on the previous rank
    p = make_plan(2, 1, 300, 50, 1, [0, 280, 600])
    assert (only(p).owner, only(p).pos_start, only(p).n) == (0, 280, 1)
    assert [(h.pos_start, h.length) for h in p.halo_recv] == [(281, 19)]


def test_sink_tokens_that_straddle_a_chunk_boundary_travel_in_pieces():
    # cp=3, S=6, W=3, two sink tokens, the last sequence starts at 5: its sinks are tokens 5 (rank 0) and
    # 6 (rank 1); rank 2 needs both and neither is inside its window
    p = make_plan(3, 2, 6, 3, 2, [0, 1, 3, 5, 18])
    assert [(s.owner, s.pos_start, s.n) for s in p.sink_recv] == [(0, 5, 1), (1, 6, 1)]
    assert [(h.pos_start, h.length) for h in p.halo_recv] == [(9, 3)]
    assert [(s.dst, s.offset, s.n) for s in make_plan(3, 0, 6, 3, 2, [0, 1, 3, 5, 18]).sink_send] == [(1, 5, 1), (2, 5, 1)]
    assert [(s.dst, s.offset, s.n) for s in make_plan(3, 1, 6, 3, 2, [0, 1, 3, 5, 18]).sink_send] == [(2, 0, 1)]
    # more sink tokens than a chunk holds
    p = make_plan(4, 3, 4, 2, 9, None)
    assert [(s.owner, s.pos_start, s.n) for s in p.sink_recv] == [(0, 0, 4), (1, 4, 4), (2, 8, 1)]
    assert [(h.pos_start, h.length) for h in p.halo_recv] == [(10, 2)]


def _visible_keys(p, cu, W, n_sink):
    """Keys query position p sees, from the mask definition."""
    if cu is None:
        s = 0
    else:
        s = max(c for c in cu if c <= p)
    return {t for t in range(s, p + 1) if p - t <= W or t < s + n_sink}


def test_plan_covers_every_visible_key_exactly_once():
    """Brute force over random geometries: local chunk + halos + sink pieces hold every key any local
    query sees, no position twice, and the tiles declared halo-free really need no halo."""
    import random
    rng = random.Random(7)
    for trial in range(1500):
        cp = rng.randint(1, 5)
        S = rng.choice([1, 2, 3, 6, 8, 16])
        W = rng.randint(0, 3 * S + 2)
        n_sink = rng.choice([0, 1, 2, 3, 5])
        T = cp * S
        if rng.random() < 0.5:
            cu = None
        else:
            cuts = sorted(rng.sample(range(1, T), min(T - 1, rng.randint(0, 4)))) if T > 1 else []
            cu = [0] + cuts + [T]
        for r in range(cp):
            plan = make_plan(cp, r, S, W, n_sink, cu)
            have = list(range(r * S, (r + 1) * S))
            for h in plan.halo_recv:
                assert h.src == r - h.hop and (r - h.hop) * S <= h.pos_start and h.pos_start + h.length == (r - h.hop + 1) * S
                have += range(h.pos_start, h.pos_start + h.length)
            for sr in plan.sink_recv:
                assert sr.owner * S <= sr.pos_start and sr.pos_start + sr.n <= (sr.owner + 1) * S
                have += range(sr.pos_start, sr.pos_start + sr.n)
            assert len(have) == len(set(have)), (cp, r, S, W, n_sink, cu)
            need = set()
            for p in range(r * S, (r + 1) * S):
                need |= _visible_keys(p, cu, W, n_sink)
            assert need <= set(have), (cp, r, S, W, n_sink, cu, sorted(need - set(have)))
            near = set(range(r * S, (r + 1) * S))
            for sr in plan.sink_recv:
                near |= set(range(sr.pos_start, sr.pos_start + sr.n))
            for p in range(r * S + plan.halo_tile_end * 128, (r + 1) * S):
                assert _visible_keys(p, cu, W, n_sink) <= near


def test_unequal_chunks_cover_every_visible_key_and_sends_mirror_receives():
    """Chunks of different lengths per rank (cp_chunk_lens of the varlen functions; the reference assumes
    equal ones, ring_swa/sliding_window/varlen.py:56-59): the same brute-force coverage check on the
    chunk bounds, and every receive of one rank is some other rank's send of the same tokens."""
    import random
    rng = random.Random(11)
    for trial in range(1500):
        cp = rng.randint(1, 5)
        lens = [rng.choice([1, 2, 3, 5, 8, 13]) for _ in range(cp)]
        bounds = [sum(lens[:i]) for i in range(cp + 1)]
        T = bounds[-1]
        W = rng.randint(0, T + 2)
        n_sink = rng.choice([0, 1, 2, 3, 5])
        cuts = sorted(rng.sample(range(1, T), min(T - 1, rng.randint(0, 4)))) if T > 1 else []
        cu = [0] + cuts + [T]
        plans = [make_plan(cp, r, lens[r], W, n_sink, cu, lens) for r in range(cp)]
        for r, plan in enumerate(plans):
            assert plan.q_pos_start == bounds[r] and plan.seq_per_rank == lens[r]
            have = list(range(bounds[r], bounds[r + 1]))
            for h in plan.halo_recv:
                assert h.src == r - h.hop and bounds[h.src] <= h.pos_start and h.pos_start + h.length == bounds[h.src + 1]
                have += range(h.pos_start, h.pos_start + h.length)
                assert any(s.dst == r and s.hop == h.hop and s.length == h.length for s in plans[h.src].halo_send)
            for sr in plan.sink_recv:
                assert bounds[sr.owner] <= sr.pos_start and sr.pos_start + sr.n <= bounds[sr.owner + 1]
                have += range(sr.pos_start, sr.pos_start + sr.n)
                assert any(s.dst == r and s.offset == sr.pos_start - bounds[sr.owner] and s.n == sr.n
                           for s in plans[sr.owner].sink_send)
            assert sum(len(q.halo_send) for q in plans) == sum(len(q.halo_recv) for q in plans)
            assert sum(len(q.sink_send) for q in plans) == sum(len(q.sink_recv) for q in plans)
            assert len(have) == len(set(have)), (lens, r, W, n_sink, cu)
            need = set()
            for p_ in range(bounds[r], bounds[r + 1]):
                need |= _visible_keys(p_, cu, W, n_sink)
            assert need <= set(have), (lens, r, W, n_sink, cu, sorted(need - set(have)))
            near = set(range(bounds[r], bounds[r + 1]))
            for sr in plan.sink_recv:
                near |= set(range(sr.pos_start, sr.pos_start + sr.n))
            for p_ in range(bounds[r] + plan.halo_tile_end * 128, bounds[r + 1]):
                assert _visible_keys(p_, cu, W, n_sink) <= near
    with pytest.raises(ValueError):
        make_plan(3, 1, 5, 4, 0, None, [5, 6, 5])      # this rank's length contradicts the list
    with pytest.raises(ValueError):
        make_plan(3, 1, 5, 4, 0, None, [5, 5])         # one length per rank
    with pytest.raises(ValueError):
        make_plan(3, 1, 5, 4, 0, None, [5, 5, 0])      # empty chunks are not supported


def test_rejects_bad_geometry():
    with pytest.raises(ValueError):
        make_plan(4, 4, 16, 5, 0, None)
    with pytest.raises(ValueError):
        make_plan(2, 0, 0, 5, 0, None)


def test_chunk_lens_must_add_up_to_the_packed_axis():
    """cp_chunk_lens is checked where the reference checks its equal share (before any work is queued)."""
    import torch
    import ring_swa
    q = torch.zeros(6, 2, 8)
    cu = torch.tensor([0, 4, 10], dtype=torch.int32)
    for fn in (ring_swa.ring_sliding_window_attn_varlen, ring_swa.ring_streaming_llm_attn_varlen):
        with pytest.raises(AssertionError, match="cp_chunk_lens does not add up"):
            fn(q, q, q, 3, cu, cp_size=2, cp_chunk_lens=[6, 5])


def test_peer_slots_hold_every_halo_message():
    """The receive slots of the peer-store exchange are sized from the largest and the smallest chunk only
    (every rank must come to the same layout): no halo message of any rank's plan may be larger than the
    slot of its hop, forward (16-bit K/V) or backward (gradients, float32 at most), and no plan may need a
    hop without a slot."""
    import random
    from ring_swa._peer import MAX_HOPS, slot_bytes_for
    rng = random.Random(5)
    B, hkv, D = 2, 3, 128
    for trial in range(2000):
        cp = rng.randint(2, 6)
        if rng.random() < 0.4:
            lens = [rng.choice([1, 2, 5, 8, 16])] * cp
        else:
            lens = [rng.choice([1, 2, 3, 5, 8, 13, 16]) for _ in range(cp)]
        W = rng.randint(0, sum(lens) + 2)
        cuts = sorted(rng.sample(range(1, sum(lens)), rng.randint(0, 3))) if sum(lens) > 3 else []
        cu = [0] + cuts + [sum(lens)]
        slots = slot_bytes_for(cp, max(lens), W, B, hkv, D, min(lens))
        plans = [make_plan(cp, r, lens[r], W, 0, cu, lens) for r in range(cp)]
        top = max([h.hop for p in plans for h in p.halo_recv], default=0)
        if slots is None:
            assert top == 0 or (W + min(lens) - 1) // min(lens) > MAX_HOPS
            continue
        assert top <= len(slots), (lens, W, cu)
        for p in plans:
            for h in p.halo_recv:
                assert 2 * B * h.length * hkv * D * 4 <= slots[h.hop - 1], (lens, W, cu, h)
