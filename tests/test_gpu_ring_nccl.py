"""The ring path on real GPUs (NCCL, one process per GPU).  Skipped on a single-GPU box."""
import json
import os
import tempfile

import pytest
import torch
import torch.multiprocessing as mp

from oracle.dense_attn import dense_attn_fwd_bwd
from ring_cases import make_inputs, run_rank

pytestmark = pytest.mark.gpu


def _job(fn, T, B, hq, hkv, W, seed, cu=None, n_sink=0, chunk_lens=None):
    varlen = cu is not None
    q, k, v, do = make_inputs(seed, T, hq, hkv, 128, True, None if varlen else B, None)
    q4, k4, v4, do4 = (x.unsqueeze(0) if varlen else x for x in (q, k, v, do))
    o, _l, dq, dk, dv = dense_attn_fwd_bwd(q4, k4, v4, do4, W, None, n_sink, cu)
    exp = {"out": o, "dq": dq, "dk": dk, "dv": dv}
    if varlen:
        exp = {k_: v_.squeeze(0) for k_, v_ in exp.items()}
    return dict(fn=fn, T=T, B=B, hq=hq, hkv=hkv, d=128, W=W, seed=seed, cu=cu, n_sink=n_sink, bf16_grid=True,
                chunk_lens=chunk_lens, dtype=torch.bfloat16, expect={k_: v_.float().numpy() for k_, v_ in exp.items()})


def _worker(rank, ws, port, jobs, outdir, halo):
    torch.cuda.set_device(rank)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    os.environ["RING_SWA_HALO"] = halo
    run_rank(rank, ws, port, jobs, outdir, device=f"cuda:{rank}")


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("halo", ["peer", "nccl"])
def test_ring_on_gpus_matches_oracle(halo):
    """Both ways the halos travel: peer stores into the receiver's buffer (the default between GPUs) and
    torch.distributed point-to-point messages."""
    ws = min(4, torch.cuda.device_count())
    ws = 4 if ws >= 4 else 2
    T = 1024 * ws
    uneven = [1024] * ws          # chunks of different lengths: 1300, 748, 1024, ...
    uneven[0] += 276
    uneven[1] -= 276
    jobs = [
        _job("ring_sliding_window_attn", T, 2, 4, 2, 300, 61),
        _job("ring_sliding_window_attn", T, 1, 4, 4, 1500, 62),            # W >= S: merge path
        _job("ring_streaming_llm_attn", T, 1, 4, 1, 200, 63, n_sink=1),
        _job("ring_sliding_window_attn_varlen", T, None, 4, 2, 400, 64, cu=[0, 700, 701, T - 300, T]),
        _job("ring_streaming_llm_attn_varlen", T, None, 4, 2, 150, 65, cu=[0, 900, T], n_sink=1),
        _job("ring_sliding_window_attn_varlen", T, None, 4, 2, 400, 66, cu=[0, 700, 1300, T], chunk_lens=uneven),
        _job("ring_streaming_llm_attn_varlen", T, None, 4, 1, 900, 67, cu=[0, 1200, T], n_sink=2, chunk_lens=uneven),
    ]
    with tempfile.TemporaryDirectory() as tmp:
        mp.spawn(_worker, args=(ws, 29771 if halo == "peer" else 29773, jobs, tmp, halo), nprocs=ws, join=True)
        res = [json.load(open(os.path.join(tmp, f"r{r}.json"))) for r in range(ws)]
    for r, per_rank in enumerate(res):
        for job, errs in zip(jobs, per_rank):
            for name in ("out", "dq", "dk", "dv"):
                assert errs[name] <= 2e-2 + 1e-2 * errs[name + "_ref_max"], f"rank {r} {job['fn']} {name}: {errs}"
