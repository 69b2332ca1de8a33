"""Generates the golden vectors under tests/golden/ from the REFERENCE's own code.

Run once, on a machine that has the reference project checked out, with its
location in ``$RSWA_REFERENCE``::

    RSWA_REFERENCE=<checkout of ring-sliding-window-attention> python tests/golden/make_golden.py

Two sources, both executed on CPU:

1. The reference's dense test oracles, imported unmodified
   (test/test_local_swa.py:7-95, test/test_local_slm.py:7-73).
2. The reference's ring autograd functions, imported unmodified and run on
   ``gloo`` CPU ranks.  Their third-party boundary (the flash-attn wrappers of
   ring_swa/ops/wrap_flash.py:168-429, which have no CPU kernel) is rebound to a
   dense restatement with flash-attn's documented bottom-right aligned window
   semantics (stated at test/test_local_swa.py:56-89); the Triton merge is rebound
   to the reference's own torch merge (ring_swa/ops/merge.py:16-50) and the
   all_to_all of ring_swa/ops/comm.py:102-149 (not implemented by gloo) to an
   all_gather with the same result.

The outputs are what the four public functions return (and the grads they
produce) for a global sequence sharded over cp ranks; they are written as small
``.npz`` files next to this script.  Nothing here is imported by the product.
"""
from __future__ import annotations

import importlib.util
import os
import sys
import tempfile

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

REF = os.environ.get("RSWA_REFERENCE", "")
if not REF or not os.path.isdir(os.path.join(REF, "ring_swa")):
    raise SystemExit("set RSWA_REFERENCE to a checkout of the reference project (it must contain ring_swa/)")
HERE = os.path.dirname(os.path.abspath(__file__))


# --------------------------------------------------------------------------------------
# dense stand-ins for the flash-attn boundary
# --------------------------------------------------------------------------------------
def _mask(sq, sk, window, causal):
    wl, wr = window
    if causal:
        wr = 0
    i = torch.arange(sq)[:, None]
    j = torch.arange(sk)[None, :]
    rel = j - i
    off = sk - sq
    m = torch.ones(sq, sk, dtype=torch.bool)
    if wl >= 0:
        m &= rel >= off - wl
    if wr >= 0:
        m &= rel <= off + wr
    return m


def _rep(x, g):
    return x if g == 1 else x.repeat_interleave(g, dim=2)


def dense_fwd(q, k, v, softmax_scale, window_size, causal):
    B, sq, hq, d = q.shape
    sk, hk = k.shape[1], k.shape[2]
    g = hq // hk
    m = _mask(sq, sk, tuple(window_size), causal)
    s = torch.einsum("bihd,bjhd->bhij", q.float(), _rep(k, g).float()) * softmax_scale
    s = s.masked_fill(~m[None, None], float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    safe = torch.where(torch.isinf(lse), torch.zeros_like(lse), lse)
    p = torch.exp(s - safe[..., None]).masked_fill(~m[None, None], 0.0)
    out = torch.einsum("bhij,bjhd->bihd", p, _rep(v, g).float())
    return out.to(q.dtype), lse.float()


def dense_bwd(q, k, v, o, softmax_lse, do, dq, dk, dv, softmax_scale, window_size, causal):
    B, sq, hq, d = q.shape
    sk, hk = k.shape[1], k.shape[2]
    g = hq // hk
    m = _mask(sq, sk, tuple(window_size), causal)
    kr, vr = _rep(k, g).float(), _rep(v, g).float()
    s = torch.einsum("bihd,bjhd->bhij", q.float(), kr) * softmax_scale
    p = torch.exp(s - softmax_lse.float()[..., None]).masked_fill(~m[None, None], 0.0)
    dof = do.float()
    dvr = torch.einsum("bhij,bihd->bjhd", p, dof)
    dp = torch.einsum("bihd,bjhd->bhij", dof, vr)
    delta = (dof * o.float()).sum(-1).permute(0, 2, 1)  # [B,H,Sq]
    ds = p * (dp - delta[..., None])
    dqf = torch.einsum("bhij,bjhd->bihd", ds, kr) * softmax_scale
    dkr = torch.einsum("bhij,bihd->bjhd", ds, q.float()) * softmax_scale
    dq.copy_(dqf.to(dq.dtype))
    dk.copy_(dkr.reshape(B, sk, hk, g, d).sum(3).to(dk.dtype))
    dv.copy_(dvr.reshape(B, sk, hk, g, d).sum(3).to(dv.dtype))


def dense_fwd_varlen(q, k, v, softmax_scale, window_size, cu_seqlens_q, cu_seqlens_k,
                     max_seqlen_q, max_seqlen_k, causal):
    T, hq, d = q.shape
    out = torch.zeros_like(q)
    lse = torch.full((hq, T), float("-inf"), dtype=torch.float32)
    cq, ck = cu_seqlens_q.tolist(), cu_seqlens_k.tolist()
    for a in range(len(cq) - 1):
        qs, qe, ks, ke = cq[a], cq[a + 1], ck[a], ck[a + 1]
        if qe == qs:
            continue
        o_, l_ = dense_fwd(q[None, qs:qe], k[None, ks:ke], v[None, ks:ke], softmax_scale,
                           window_size, causal)
        out[qs:qe] = o_[0]
        lse[:, qs:qe] = l_[0]
    return out, lse


def dense_bwd_varlen(q, k, v, o, softmax_lse, do, dq, dk, dv, softmax_scale, window_size,
                     cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, causal):
    cq, ck = cu_seqlens_q.tolist(), cu_seqlens_k.tolist()
    dq.zero_(), dk.zero_(), dv.zero_()
    for a in range(len(cq) - 1):
        qs, qe, ks, ke = cq[a], cq[a + 1], ck[a], ck[a + 1]
        if qe == qs:
            continue
        dq_ = torch.zeros_like(dq[None, qs:qe])
        dk_ = torch.zeros_like(dk[None, ks:ke])
        dv_ = torch.zeros_like(dv[None, ks:ke])
        dense_bwd(q[None, qs:qe], k[None, ks:ke], v[None, ks:ke], o[None, qs:qe],
                  softmax_lse[None, :, qs:qe], do[None, qs:qe], dq_, dk_, dv_,
                  softmax_scale, window_size, causal)
        dq[qs:qe] = dq_[0]
        dk[ks:ke] = dk_[0]
        dv[ks:ke] = dv_[0]


def _gather_exchange(tensor_to_send, send_to_rank, cp_group):
    """all_gather restatement of ring_swa/ops/comm.py:102-149 for gloo."""
    ws = dist.get_world_size(group=cp_group)
    me = dist.get_rank(group=cp_group)
    dst = torch.tensor([int(send_to_rank)], dtype=torch.long)
    dsts = [torch.zeros_like(dst) for _ in range(ws)]
    bufs = [torch.zeros_like(tensor_to_send) for _ in range(ws)]
    dist.all_gather(dsts, dst, group=cp_group)
    dist.all_gather(bufs, tensor_to_send.contiguous(), group=cp_group)
    out = torch.zeros_like(tensor_to_send)
    for r in range(ws):
        if int(dsts[r]) == me:
            out += bufs[r]
    return out


def import_reference():
    sys.path.insert(0, REF)
    import ring_swa  # noqa: F401  (the reference package)
    import ring_swa.ops.attn as attn
    import ring_swa.ops.merge as merge
    import ring_swa.streaming_llm.naive as naive
    import ring_swa.streaming_llm.nonvarlen as slm_nv
    import ring_swa.streaming_llm.varlen as slm_vl

    attn.wrapped_flash_attn_fwd = dense_fwd
    attn.wrapped_flash_attn_bwd = dense_bwd
    attn.wrapped_flash_attn_fwd_varlen = dense_fwd_varlen
    attn.wrapped_flash_attn_bwd_varlen = dense_bwd_varlen
    naive.wrapped_flash_attn_fwd = dense_fwd
    naive.wrapped_flash_attn_bwd = dense_bwd
    naive.wrapped_flash_attn_fwd_varlen = dense_fwd_varlen
    naive.wrapped_flash_attn_bwd_varlen = dense_bwd_varlen
    attn.merge_attn_out = merge.torch_merge_attn_out
    naive.merge_attn_out = merge.torch_merge_attn_out
    slm_nv.merge_attn_out = merge.torch_merge_attn_out
    slm_vl.exchange_and_sum_tensors = _gather_exchange
    return ring_swa


def load_test_module(name):
    spec = importlib.util.spec_from_file_location(name, os.path.join(REF, "test", name + ".py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


# --------------------------------------------------------------------------------------
# ring cases
# --------------------------------------------------------------------------------------
def make_inputs(seed, T, hq, hkv, d, bf16_grid, batch=None, sink_rows=None):
    """q, k, v, dO ~ N(0,1) drawn in that order from torch.manual_seed(seed).

    ``bf16_grid`` rounds the draws to bf16-representable values so that a bf16
    kernel sees bit-identical inputs.  ``sink_rows`` overwrites q/k/v at the given
    row indices with row 0's content (the identical-sink assumption of the
    StreamingLLM varlen path, test/test_ring_slm_varlen.py:145-147).
    """
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


def _rank_main(rank, cp, fn_name, case, tmpdir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(case["port"])
    torch.set_num_threads(1)
    dist.init_process_group("gloo", rank=rank, world_size=cp)
    ring_swa = import_reference()
    group = dist.group.WORLD
    varlen = "varlen" in fn_name
    sink_rows = case.get("sink_rows")
    q, k, v, do = make_inputs(case["seed"], case["T"], case["hq"], case["hkv"], case["d"],
                              case["bf16_grid"], None if varlen else case["B"], sink_rows)
    S = case["T"] // cp
    sl = (slice(rank * S, (rank + 1) * S),) if varlen else (slice(None), slice(rank * S, (rank + 1) * S))
    ql, kl, vl, dol = (x[sl].clone() for x in (q, k, v, do))
    ql.requires_grad_(True), kl.requires_grad_(True), vl.requires_grad_(True)
    fn = getattr(ring_swa, fn_name)
    kw = dict(window_size=case["W"], cp_group=group, cp_size=cp, cp_local_rank=rank)
    if varlen:
        kw["cu_seqlens"] = torch.tensor(case["cu"], dtype=torch.int32)
    out = fn(ql, kl, vl, **kw)
    out.backward(dol)
    torch.save({"out": out.detach(), "dq": ql.grad, "dk": kl.grad, "dv": vl.grad},
               os.path.join(tmpdir, f"r{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


def run_ring_case(fn_name, cp, case):
    with tempfile.TemporaryDirectory() as tmp:
        mp.spawn(_rank_main, args=(cp, fn_name, case, tmp), nprocs=cp, join=True)
        parts = [torch.load(os.path.join(tmp, f"r{r}.pt")) for r in range(cp)]
    dim = 0 if "varlen" in fn_name else 1
    return {k: torch.cat([p[k] for p in parts], dim=dim) for k in ("out", "dq", "dk", "dv")}


def cu_from_lens(lens):
    cu = [0]
    for L in lens:
        cu.append(cu[-1] + L)
    return cu


PIN_W = [1, 5, 15, 16, 17, 31, 32, 33, 47, 48, 49, 63, 100]
PIN_LAYOUTS = [
    [64],
    [16, 48],
    [1, 15, 16, 32],
    [7, 1, 1, 23, 32],
    [33, 31],
    [20, 20, 24],
    [5, 40, 3, 16],
]
PIN_W_VARLEN = [3, 15, 16, 17, 30, 33, 100]


def build_pin_cases():
    """Small fp32 cases (cp=4, S=16/rank, D=8) that pin the semantics exactly."""
    port = 29610
    cases = []
    for fn in ("ring_sliding_window_attn", "ring_streaming_llm_attn"):
        for W in PIN_W:
            port += 1
            cases.append((fn, 4, dict(seed=100 + W, T=64, B=1, hq=4, hkv=2, d=8, W=W,
                                      bf16_grid=False, port=port)))
    # B = 2 is only defined for the sliding-window function (the reference's
    # StreamingLLM ring takes the sink from batch row 0 for every row)
    port += 1
    cases.append(("ring_sliding_window_attn", 2,
                  dict(seed=7, T=32, B=2, hq=4, hkv=4, d=8, W=20, bf16_grid=False, port=port)))
    for fn in ("ring_sliding_window_attn_varlen", "ring_streaming_llm_attn_varlen"):
        for li, lens in enumerate(PIN_LAYOUTS):
            for W in PIN_W_VARLEN:
                port += 1
                cu = cu_from_lens(lens)
                c = dict(seed=1000 + 10 * li + W, T=64, hq=4, hkv=2, d=8, W=W, cu=cu,
                         bf16_grid=False, port=port)
                if "streaming" in fn:
                    c["sink_rows"] = cu[:-1]
                cases.append((fn, 4, c))
    return cases


def build_gpu_cases():
    """D = 128 cases on the bf16 grid, for the CUDA kernels (outputs stored as fp16)."""
    port = 29900
    cases = []
    defs = [
        ("ring_sliding_window_attn", 2, dict(T=384, B=1, hq=2, hkv=1, W=100)),
        ("ring_sliding_window_attn", 4, dict(T=512, B=1, hq=2, hkv=2, W=300)),
        ("ring_streaming_llm_attn", 2, dict(T=384, B=1, hq=2, hkv=1, W=64)),
        ("ring_streaming_llm_attn", 4, dict(T=512, B=1, hq=2, hkv=1, W=200)),
        ("ring_sliding_window_attn_varlen", 2, dict(T=384, hq=2, hkv=1, W=90, lens=[100, 1, 155, 128])),
        ("ring_sliding_window_attn_varlen", 4, dict(T=512, hq=2, hkv=1, W=150, lens=[300, 40, 172])),
        ("ring_streaming_llm_attn_varlen", 2, dict(T=384, hq=2, hkv=1, W=50, lens=[130, 200, 54])),
        ("ring_streaming_llm_attn_varlen", 4, dict(T=512, hq=2, hkv=1, W=140, lens=[290, 222])),
    ]
    for i, (fn, cp, c) in enumerate(defs):
        port += 1
        c = dict(c, seed=500 + i, d=128, bf16_grid=True, port=port)
        if "lens" in c:
            c["cu"] = cu_from_lens(c.pop("lens"))
            if "streaming" in fn:
                c["sink_rows"] = c["cu"][:-1]
        cases.append((fn, cp, c))
    return cases


def pack_case(fn, cp, case, res, store_dtype):
    d = {"fn": fn, "cp": cp}
    for k_, v_ in case.items():
        if k_ != "port":
            d["p_" + k_] = np.asarray(v_)
    for k_, v_ in res.items():
        d[k_] = v_.numpy().astype(store_dtype)
    return d


def main():
    torch.set_num_threads(2)
    # (1) reference dense oracles, imported unmodified
    import_reference()
    swa = load_test_module("test_local_swa")
    slm = load_test_module("test_local_slm")
    dense = {}
    for i, (W, hq, hkv) in enumerate([(128, 4, 4), (17, 4, 2), (1, 2, 1), (300, 4, 1)]):
        torch.manual_seed(40 + i)
        q = torch.randn(1, 256, hq, 16)
        k = torch.randn(1, 256, hkv, 16)
        v = torch.randn(1, 256, hkv, 16)
        dense[f"swa{i}_params"] = np.array([W, hq, hkv, 40 + i])
        dense[f"swa{i}_out"] = swa.torch_sliding_window_attn_nonvarlen(q, k, v, (W, 0)).numpy()
        dense[f"slm{i}_out"] = slm.torch_streaming_llm_attn_nonvarlen(q, k, v, W).numpy()
    np.savez_compressed(os.path.join(HERE, "ref_dense_oracles.npz"), **dense)

    # (2) reference ring functions on gloo ranks
    pins = {}
    for n, (fn, cp, case) in enumerate(build_pin_cases()):
        res = run_ring_case(fn, cp, case)
        for k_, v_ in pack_case(fn, cp, case, res, np.float32).items():
            pins[f"c{n:03d}_{k_}"] = v_
        print("pin", n, fn, case["W"], case.get("cu"), flush=True)
    np.savez_compressed(os.path.join(HERE, "ref_ring_pins.npz"), **pins)

    for n, (fn, cp, case) in enumerate(build_gpu_cases()):
        res = run_ring_case(fn, cp, case)
        np.savez_compressed(os.path.join(HERE, f"ref_ring_d128_{n}.npz"),
                            **pack_case(fn, cp, case, res, np.float16))
        print("d128", n, fn, flush=True)


if __name__ == "__main__":
    main()
