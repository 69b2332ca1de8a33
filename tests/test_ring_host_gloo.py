"""The ring host logic (halo plan, exchange, phase split, merge path, gradient routing) on gloo CPU
ranks, with the CUDA entry points replaced by oracle-backed stand-ins (tests/cpu_backend.py).

Checked against (a) the reference's own ring functions' outputs (tests/golden/ref_ring_pins.npz,
cp = 4) and (b) the dense oracle on the global sequence (cp = 2, shapes that exercise query-tile
phase splitting, W >= S with the merge path, batch > 1 and more than one sink token).
"""
import json
import os
import tempfile

import pytest
import torch
import torch.multiprocessing as mp

from oracle.dense_attn import dense_attn_fwd_bwd
from ring_cases import case_params, load_pins, make_inputs, run_rank

TOL = 2e-5


def _spawn(ws, port, jobs):
    with tempfile.TemporaryDirectory() as tmp:
        mp.spawn(run_rank, args=(ws, port, jobs, tmp), nprocs=ws, join=True)
        return [json.load(open(os.path.join(tmp, f"r{r}.json"))) for r in range(ws)]


def _assert_small(results, jobs, tol):
    for r, per_rank in enumerate(results):
        for job, errs in zip(jobs, per_rank):
            for name in ("out", "dq", "dk", "dv"):
                assert errs[name] <= tol * max(1.0, errs[name + "_ref_max"]), (
                    f"rank {r} {job['fn']} W={job['W']} cu={job.get('cu')} {name}: {errs}")


@pytest.mark.timeout(900)
def test_ring_matches_reference_pins_cp4():
    jobs = []
    for c in load_pins():
        if int(c["cp"]) != 4:
            continue
        p = case_params(c)
        job = dict(p, fn=str(c["fn"]), expect={k: c[k] for k in ("out", "dq", "dk", "dv")})
        jobs.append(job)
    assert len(jobs) > 100
    res = _spawn(4, 29731, jobs)
    _assert_small(res, jobs, TOL)


def _dense_job(fn, T, B, hq, hkv, d, W, seed, cu=None, n_sink=0, chunk_lens=None):
    varlen = cu is not None
    sink_rows = None
    q, k, v, do = make_inputs(seed, T, hq, hkv, d, False, None if varlen else B, sink_rows)
    q4, k4, v4, do4 = (x.unsqueeze(0) if varlen else x for x in (q, k, v, do))
    o, _l, dq, dk, dv = dense_attn_fwd_bwd(q4, k4, v4, do4, W, None, n_sink, cu, compute_dtype=torch.float64)
    exp = {"out": o, "dq": dq, "dk": dk, "dv": dv}
    if varlen:
        exp = {k_: v_.squeeze(0) for k_, v_ in exp.items()}
    return dict(fn=fn, T=T, B=B, hq=hq, hkv=hkv, d=d, W=W, seed=seed, cu=cu, n_sink=n_sink, bf16_grid=False,
                chunk_lens=chunk_lens, expect={k_: v_.float().numpy() for k_, v_ in exp.items()})


@pytest.mark.timeout(600)
def test_ring_matches_dense_oracle_cp2():
    jobs = [
        # phase split: tiles [1,3) local only, tile 0 with halo
        _dense_job("ring_sliding_window_attn", 600, 1, 2, 1, 8, 100, 11),
        _dense_job("ring_sliding_window_attn", 600, 2, 2, 2, 8, 129, 12),
        # W >= S: halo as a second partial + merge
        _dense_job("ring_sliding_window_attn", 520, 1, 2, 1, 8, 300, 13),
        _dense_job("ring_sliding_window_attn", 64, 2, 4, 2, 8, 1000, 14),
        # StreamingLLM with the sink remote, several sinks, each batch row its own sink
        _dense_job("ring_streaming_llm_attn", 600, 1, 2, 1, 8, 60, 15, n_sink=1),
        _dense_job("ring_streaming_llm_attn", 600, 2, 2, 1, 8, 60, 16, n_sink=4),
        _dense_job("ring_streaming_llm_attn", 64, 1, 2, 1, 8, 40, 17, n_sink=3),
        # packed sequences: boundary on the rank edge, one-token sequences, long crossing sequence
        _dense_job("ring_sliding_window_attn_varlen", 600, None, 2, 1, 8, 70, 18, cu=[0, 300, 301, 420, 600]),
        _dense_job("ring_sliding_window_attn_varlen", 600, None, 2, 1, 8, 400, 19, cu=[0, 10, 600]),
        _dense_job("ring_streaming_llm_attn_varlen", 600, None, 2, 1, 8, 50, 20, cu=[0, 130, 500, 600], n_sink=1),
        _dense_job("ring_streaming_llm_attn_varlen", 600, None, 2, 2, 8, 50, 21, cu=[0, 130, 500, 600], n_sink=2),
        # the sink of the crossing sequence lies inside the window's reach on the previous rank, while the
        # later query tiles of this rank run before the halo arrives
        _dense_job("ring_streaming_llm_attn_varlen", 600, None, 2, 1, 8, 50, 22, cu=[0, 280, 600], n_sink=1),
        _dense_job("ring_streaming_llm_attn", 600, 1, 2, 1, 8, 400, 23, n_sink=2),
    ]
    res = _spawn(2, 29741, jobs)
    _assert_small(res, jobs, TOL)


@pytest.mark.timeout(600)
def test_sink_tokens_on_two_ranks_cp3():
    """The first tokens of a sequence that starts just before a chunk boundary lie on two ranks; a
    later rank gets them as two pieces and returns their gradients to both owners."""
    jobs = [
        _dense_job("ring_streaming_llm_attn_varlen", 600, None, 2, 1, 8, 40, 31, cu=[0, 199, 600], n_sink=3),
        _dense_job("ring_streaming_llm_attn_varlen", 600, None, 2, 2, 8, 70, 32, cu=[0, 50, 398, 600], n_sink=5),
        _dense_job("ring_streaming_llm_attn", 12, 1, 2, 1, 8, 2, 33, n_sink=9),   # more sink tokens than a chunk holds
    ]
    res = _spawn(3, 29751, jobs)
    _assert_small(res, jobs, TOL)


@pytest.mark.timeout(600)
def test_chunks_of_different_lengths_cp3():
    """cp_chunk_lens: the packed token axis cut into unequal shares (at sequence boundaries, inside
    sequences, a chunk shorter than the window so that the halo comes from two ranks, a one-token
    chunk), against the dense oracle on the global sequence."""
    V, SV = "ring_sliding_window_attn_varlen", "ring_streaming_llm_attn_varlen"
    jobs = [
        _dense_job(V, 600, None, 2, 1, 8, 70, 41, cu=[0, 150, 420, 600], chunk_lens=[150, 270, 180]),   # cut at sequence starts
        _dense_job(V, 600, None, 2, 2, 8, 90, 42, cu=[0, 100, 600], chunk_lens=[310, 40, 250]),        # W > middle chunk: two hops
        _dense_job(V, 600, None, 2, 1, 8, 700, 43, cu=[0, 600], chunk_lens=[1, 399, 200]),            # W >= T, one-token chunk
        _dense_job(V, 600, None, 2, 1, 8, 130, 44, cu=[0, 290, 291, 600], chunk_lens=[200, 100, 300]),
        _dense_job(SV, 600, None, 2, 1, 8, 50, 45, cu=[0, 130, 500, 600], n_sink=1, chunk_lens=[128, 272, 200]),
        _dense_job(SV, 600, None, 2, 2, 8, 60, 46, cu=[0, 199, 600], n_sink=3, chunk_lens=[200, 150, 250]),   # sink pieces on two ranks
    ]
    res = _spawn(3, 29761, jobs)
    _assert_small(res, jobs, TOL)


@pytest.mark.timeout(600)
def test_reference_class_names_cp2():
    """RingSlidingWindowAttn.apply(...) and its three siblings take the reference's positional arguments
    (ring_swa/sliding_window/nonvarlen.py:17-32, varlen.py:19-36, streaming_llm/nonvarlen.py:20-35,
    varlen.py:20-37) and give the ring functions' results."""
    jobs = [
        dict(_dense_job("ring_sliding_window_attn", 600, 1, 2, 1, 8, 100, 51), cls="sliding_window.nonvarlen:RingSlidingWindowAttn"),
        dict(_dense_job("ring_sliding_window_attn_varlen", 600, None, 2, 1, 8, 70, 52, cu=[0, 300, 301, 420, 600]),
             cls="sliding_window.varlen:RingSlidingWindowAttnVarlen"),
        dict(_dense_job("ring_streaming_llm_attn", 600, 1, 2, 1, 8, 60, 53, n_sink=1), cls="streaming_llm.nonvarlen:RingStreamingLLMAttn"),
        dict(_dense_job("ring_streaming_llm_attn_varlen", 600, None, 2, 1, 8, 50, 54, cu=[0, 130, 500, 600], n_sink=1),
             cls="streaming_llm.varlen:RingStreamingLLMVarlen"),
    ]
    res = _spawn(2, 29781, jobs)
    _assert_small(res, jobs, TOL)
