"""Shared helpers for the multi-rank host-logic tests (gloo, CPU)."""
import json
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
GOLDEN = os.path.join(HERE, "golden")


def make_inputs(seed, T, hq, hkv, d, bf16_grid, batch=None, sink_rows=None):
    """Same draw order as tests/golden/make_golden.py: q, k, v, dO from torch.manual_seed(seed)."""
    torch.manual_seed(seed)
    lead = (T,) if batch is None else (batch, T)
    q = torch.randn(*lead, hq, d)
    k = torch.randn(*lead, hkv, d)
    v = torch.randn(*lead, hkv, d)
    do = torch.randn(*lead, hq, d)
    if bf16_grid:
        q, k, v, do = (x.bfloat16().float() for x in (q, k, v, do))
    if sink_rows is not None:
        for x in (q, k, v):
            x[sink_rows] = x[0].clone()
    return q, k, v, do


def load_pins():
    """The reference ring outputs on small fp32 cases, as a list of dicts."""
    z = np.load(os.path.join(GOLDEN, "ref_ring_pins.npz"), allow_pickle=False)
    ids = sorted({k.split("_")[0] for k in z.files})
    cases = []
    for cid in ids:
        c = {k[len(cid) + 1:]: z[k] for k in z.files if k.startswith(cid + "_")}
        cases.append(c)
    return cases


def case_params(c):
    p = {k[2:]: c[k] for k in c if k.startswith("p_")}
    out = dict(seed=int(p["seed"]), T=int(p["T"]), hq=int(p["hq"]), hkv=int(p["hkv"]), d=int(p["d"]),
               W=int(p["W"]), bf16_grid=bool(p["bf16_grid"]))
    out["B"] = int(p["B"]) if "B" in p else None
    out["cu"] = [int(x) for x in p["cu"]] if "cu" in p else None
    out["sink_rows"] = [int(x) for x in p["sink_rows"]] if "sink_rows" in p else None
    return out


def run_rank(rank, ws, port, jobs, outdir, device="cpu"):
    """Child process body: runs every job through the public API on this rank and records the
    max abs error of out/dq/dk/dv against the expected GLOBAL arrays."""
    for p in (ROOT, os.path.join(ROOT, "ring-sliding-window-attention_b200"), HERE):
        if p not in sys.path:
            sys.path.insert(0, p)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.set_num_threads(1)
    from datetime import timedelta
    dist.init_process_group("gloo" if device == "cpu" else "nccl", rank=rank, world_size=ws,
                            timeout=timedelta(seconds=180))
    import ring_swa
    if device == "cpu":
        import cpu_backend
        cpu_backend.install()
    results = []
    for job in jobs:
        fn = getattr(ring_swa, job["fn"])
        varlen = "varlen" in job["fn"]
        q, k, v, do = make_inputs(job["seed"], job["T"], job["hq"], job["hkv"], job["d"], job["bf16_grid"],
                                  None if varlen else job["B"], job.get("sink_rows"))
        S = job["T"] // ws
        a, b = rank * S, (rank + 1) * S
        if job.get("chunk_lens"):   # chunks of different lengths (varlen functions only)
            a = sum(job["chunk_lens"][:rank])
            b = a + job["chunk_lens"][rank]
        sl = (slice(a, b),) if varlen else (slice(None), slice(a, b))
        dt = job.get("dtype", torch.float32)
        ql, kl, vl, dol = (x[sl].clone().to(device=device, dtype=dt) for x in (q, k, v, do))
        for x in (ql, kl, vl):
            x.requires_grad_(True)
        kw = dict(window_size=job["W"], cp_group=dist.group.WORLD, cp_size=ws, cp_local_rank=rank)
        if varlen:
            kw["cu_seqlens"] = torch.tensor(job["cu"], dtype=torch.int32, device=device)
        if job.get("chunk_lens"):
            kw["cp_chunk_lens"] = job["chunk_lens"]
        if job.get("n_sink", 1) != 1 and "streaming" in job["fn"]:
            kw["num_sink_tokens"] = job["n_sink"]
        if job.get("cls"):
            # through the reference's autograd class name: positional arguments in the reference's order
            import importlib
            mod, name = job["cls"].split(":")
            cls = getattr(importlib.import_module("ring_swa." + mod), name)
            pos = [ql, kl, vl, job["W"]] + ([kw["cu_seqlens"], None] if varlen else [])
            pos += [dist.group.WORLD, ws, rank, (rank - 1) % ws, (rank + 1) % ws, None, None]
            out = cls.apply(*pos)
        else:
            out = fn(ql, kl, vl, **kw)
        out.backward(dol)
        errs = {}
        for name, got in (("out", out.detach()), ("dq", ql.grad), ("dk", kl.grad), ("dv", vl.grad)):
            exp = torch.as_tensor(job["expect"][name]).float()[sl]
            errs[name] = float((got.float().cpu() - exp).abs().max())
            errs[name + "_ref_max"] = float(exp.abs().max())
        results.append(errs)
    with open(os.path.join(outdir, f"r{rank}.json"), "w") as f:
        json.dump(results, f)
    dist.barrier()
    dist.destroy_process_group()
