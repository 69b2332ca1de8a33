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
        assert p.sink_recv is None and not p.sink_send


def test_sends_mirror_receives():
    for cu in (None, [0, 7, 8, 9, 40, 64], [0, 64], [0, 16, 32, 48, 64]):
        for W in (1, 5, 16, 17, 40, 100):
            for ns in (0, 1, 3):
                plans = [make_plan(4, r, 16, W, ns, cu) for r in range(4)]
                for r, p in enumerate(plans):
                    for h in p.halo_recv:
                        assert any(s.dst == r and s.length == h.length for s in plans[h.src].halo_send)
                    if p.sink_recv is not None:
                        o = p.sink_recv.owner
                        assert any(s.dst == r and s.n == p.sink_recv.n and
                                   s.offset + o * 16 == p.sink_recv.pos_start for s in plans[o].sink_send)
                    n_recv = sum(1 for q in plans for h in q.halo_recv if h.src == r)
                    assert n_recv == len(p.halo_send)


def test_varlen_halo_stops_at_sequence_start():
    cu = [0, 30, 64]
    p = make_plan(4, 2, 16, 100, 0, cu)      # rank 2 starts at 32, its sequence at 30
    assert [(h.src, h.length, h.pos_start) for h in p.halo_recv] == [(1, 2, 30)]
    p = make_plan(4, 2, 16, 100, 0, [0, 32, 64])   # sequence starts exactly on the rank edge
    assert p.halo_recv == [] and p.halo_tile_end == 0


def test_sink_travels_separately_and_never_overlaps_the_halo():
    p = make_plan(4, 3, 16, 5, 1, None)
    assert (p.sink_recv.owner, p.sink_recv.pos_start, p.sink_recv.n) == (0, 0, 1)
    # window reaches token 0: the sink still has its own message and the halo starts behind it
    p = make_plan(4, 1, 16, 20, 1, None)
    assert (p.sink_recv.pos_start, p.sink_recv.n) == (0, 1)
    assert [(h.pos_start, h.length) for h in p.halo_recv] == [(1, 15)]
    p = make_plan(4, 1, 16, 14, 4, None)
    assert (p.sink_recv.pos_start, p.sink_recv.n) == (0, 4)
    assert [(h.pos_start, h.length) for h in p.halo_recv] == [(4, 12)]
    # the sequence starts on this rank: its sink is local, nothing extra travels
    assert make_plan(4, 2, 16, 5, 1, [0, 32, 64]).sink_recv is None
    assert make_plan(4, 0, 16, 5, 1, None).sink_recv is None
    # packed: the crossing sequence starts inside the window's reach on the previous rank
    p = make_plan(2, 1, 300, 50, 1, [0, 280, 600])
    assert (p.sink_recv.owner, p.sink_recv.pos_start, p.sink_recv.n) == (0, 280, 1)
    assert [(h.pos_start, h.length) for h in p.halo_recv] == [(281, 19)]


def test_rejects_bad_geometry():
    with pytest.raises(ValueError):
        make_plan(4, 4, 16, 5, 0, None)
    with pytest.raises(ValueError):
        make_plan(2, 0, 0, 5, 0, None)
