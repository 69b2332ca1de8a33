"""The four public functions on one GPU (cp_group=None): parity with the oracle, with the vectors the
reference's ring functions produced (tests/golden/ref_ring_d128_*.npz), and the reference's error
behaviour.  Full-size checks use properties that do not need a dense oracle."""
import glob
import os

import numpy as np
import pytest
import torch

from gpu_util import assert_close, assert_lse_close, randn_bf16
from oracle.dense_attn import dense_attn_fwd_bwd
from ring_cases import GOLDEN, case_params, make_inputs

pytestmark = pytest.mark.gpu
D = 128


def _run(fn, q, k, v, do, **kw):
    dev = torch.device("cuda")
    ql, kl, vl = (x.to(dev).requires_grad_(True) for x in (q, k, v))
    out = fn(ql, kl, vl, **kw)
    out.backward(do.to(dev))
    from ring_swa._kernels import check_device_status
    check_device_status()
    return out.detach(), ql.grad, kl.grad, vl.grad


def test_sliding_window_nonvarlen():
    import ring_swa
    q, k, v, do = (randn_bf16(2, 500, h, D, seed=s) for h, s in ((4, 1), (2, 2), (2, 3), (4, 4)))
    ro, _, rdq, rdk, rdv = dense_attn_fwd_bwd(q, k, v, do, 120)
    out, dq, dk, dv = _run(ring_swa.ring_sliding_window_attn, q, k, v, do, window_size=120)
    for n, a, b in (("out", out, ro), ("dq", dq, rdq), ("dk", dk, rdk), ("dv", dv, rdv)):
        assert_close(n, a, b)
    assert out.dtype == torch.bfloat16 and out.shape == q.shape


def test_streaming_llm_nonvarlen_and_naive_alias():
    import ring_swa
    from ring_swa.streaming_llm.naive import naive_streaming_llm_attn
    q, k, v, do = (randn_bf16(1, 700, h, D, seed=s) for h, s in ((4, 5), (1, 6), (1, 7), (4, 8)))
    ro, _, rdq, rdk, rdv = dense_attn_fwd_bwd(q, k, v, do, 64, None, 1)
    out, dq, dk, dv = _run(ring_swa.ring_streaming_llm_attn, q, k, v, do, window_size=64, softmax_scale=None)
    for n, a, b in (("out", out, ro), ("dq", dq, rdq), ("dk", dk, rdk), ("dv", dv, rdv)):
        assert_close(n, a, b)
    out2, *_ = _run(naive_streaming_llm_attn, q, k, v, do, window_size=64)
    assert torch.equal(out, out2)
    ro4, *_ = dense_attn_fwd_bwd(q, k, v, do, 64, None, 4)
    out4, *_ = _run(ring_swa.ring_streaming_llm_attn, q, k, v, do, window_size=64, num_sink_tokens=4)
    assert_close("out(4 sinks)", out4, ro4)


def test_varlen_functions():
    import ring_swa
    cu = [0, 100, 101, 400, 777]
    q, k, v, do = (randn_bf16(777, h, D, seed=s) for h, s in ((4, 9), (2, 10), (2, 11), (4, 12)))
    cud = torch.tensor(cu, dtype=torch.int32, device="cuda")
    for fn, ns in ((ring_swa.ring_sliding_window_attn_varlen, 0), (ring_swa.ring_streaming_llm_attn_varlen, 1)):
        ro, _, rdq, rdk, rdv = dense_attn_fwd_bwd(q[None], k[None], v[None], do[None], 90, 0.1, ns, cu)
        out, dq, dk, dv = _run(fn, q, k, v, do, window_size=90, cu_seqlens=cud, cp_size=1, softmax_scale=0.1)
        for n, a, b in (("out", out, ro[0]), ("dq", dq, rdq[0]), ("dk", dk, rdk[0]), ("dv", dv, rdv[0])):
            assert_close(n, a, b)
    # the single-GPU names of ring_swa/streaming_llm/naive.py (function :232 and class :90) and the ring
    # classes' apply() with the reference's positional arguments give the same tensors
    from ring_swa.sliding_window.varlen import RingSlidingWindowAttnVarlen
    from ring_swa.streaming_llm.naive import StreamingLLMAttnVarlen, naive_streaming_llm_attn_varlen
    slm, *_ = _run(ring_swa.ring_streaming_llm_attn_varlen, q, k, v, do, window_size=90, cu_seqlens=cud, cp_size=1, softmax_scale=0.1)
    a1, *_ = _run(naive_streaming_llm_attn_varlen, q, k, v, do, window_size=90, cu_seqlens=cud, softmax_scale=0.1)
    a2, *_ = _run(lambda q_, k_, v_: StreamingLLMAttnVarlen.apply(q_, k_, v_, 90, cud, 0.1), q, k, v, do)
    assert torch.equal(slm, a1) and torch.equal(slm, a2)
    swa, *_ = _run(ring_swa.ring_sliding_window_attn_varlen, q, k, v, do, window_size=90, cu_seqlens=cud, cp_size=1, softmax_scale=0.1)
    a3, *_ = _run(lambda q_, k_, v_: RingSlidingWindowAttnVarlen.apply(q_, k_, v_, 90, cud, None, None, 1, 0, None, None, None, 0.1),
                  q, k, v, do)
    assert torch.equal(swa, a3)


def test_device_side_timeout_reaches_the_host_and_clears():
    """A bounded device-side wait that runs out raises the status word; kernels launched after that do no
    work, so the host has to hear of it: the word is mirrored to pinned memory behind every backward and
    looked at when the next call starts.  The word is set from the host here (nothing on the device
    faults or waits)."""
    import ring_swa
    from ring_swa import _kernels as K
    dev = torch.device("cuda")
    q, k, v, do = (randn_bf16(1, 300, h, D, seed=s) for h, s in ((4, 61), (2, 62), (2, 63), (4, 64)))
    ro, _, rdq, rdk, rdv = dense_attn_fwd_bwd(q, k, v, do, 100)
    out, dq, dk, dv = _run(ring_swa.ring_sliding_window_attn, q, k, v, do, window_size=100)
    assert_close("out", out, ro)
    K.status_word(dev).fill_(103)                      # what a kernel whose wait ran out would leave behind
    ql, kl, vl = (x.to(dev).requires_grad_(True) for x in (q, k, v))
    ring_swa.ring_sliding_window_attn(ql, kl, vl, 100).backward(do.to(dev))   # kernels return at once
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError, match="bounded device-side wait"):
        ring_swa.ring_sliding_window_attn(ql, kl, vl, 100)
    # the report cleared the word: the next call computes again
    out, dq, dk, dv = _run(ring_swa.ring_sliding_window_attn, q, k, v, do, window_size=100)
    for n, a, b in (("out", out, ro), ("dq", dq, rdq), ("dk", dk, rdk), ("dv", dv, rdv)):
        assert_close(n, a, b)


@pytest.mark.parametrize("head_dim", [64, 96])
def test_smaller_head_dims_run_zero_padded(head_dim):
    """Head dimensions below 128 (the reference's own local tests use 1 x 1024 x 8/2 heads x 64, window 128:
    test/test_local_slm.py:76-90) run on the 128-wide kernels zero-padded; result and gradients have the
    caller's shape and match the oracle at the caller's scale."""
    import ring_swa
    q, k, v, do = (randn_bf16(1, 1024, h, head_dim, seed=s) for h, s in ((8, 71), (2, 72), (2, 73), (8, 74)))
    for fn, ns in ((ring_swa.ring_sliding_window_attn, 0), (ring_swa.ring_streaming_llm_attn, 1)):
        ro, _, rdq, rdk, rdv = dense_attn_fwd_bwd(q, k, v, do, 128, None, ns)
        out, dq, dk, dv = _run(fn, q, k, v, do, window_size=128)
        assert out.shape == q.shape and dk.shape == k.shape
        for n, a, b in (("out", out, ro), ("dq", dq, rdq), ("dk", dk, rdk), ("dv", dv, rdv)):
            assert_close(n, a, b)
    with pytest.raises(ValueError, match="head_dim"):
        ring_swa.ring_sliding_window_attn(q[..., :60].cuda(), k[..., :60].cuda(), v[..., :60].cuda(), 128)


def test_reference_error_behaviour():
    import ring_swa
    dev = "cuda"
    q = torch.zeros(256, 4, D, dtype=torch.bfloat16, device=dev)
    cu = torch.tensor([0, 256], dtype=torch.int32, device=dev)
    # ring_swa/sliding_window/varlen.py:401-403 divides by cp_size before looking at cp_group
    with pytest.raises(TypeError):
        ring_swa.ring_sliding_window_attn_varlen(q, q, q, 10, cu)
    with pytest.raises(AssertionError, match="cu_seqlens does not match"):
        ring_swa.ring_sliding_window_attn_varlen(q, q, q, 10, cu, cp_size=2)
    k3 = torch.zeros(256, 3, D, dtype=torch.bfloat16, device=dev)
    with pytest.raises(AssertionError, match="divisible"):
        ring_swa.ring_sliding_window_attn_varlen(q, k3, k3, 10, cu, cp_size=1)
    q4 = torch.zeros(1, 256, 4, D, dtype=torch.bfloat16, device=dev)
    k4 = torch.zeros(1, 128, 4, D, dtype=torch.bfloat16, device=dev)
    with pytest.raises(AssertionError, match="Sequence length must be the same"):
        ring_swa.ring_sliding_window_attn(q4, k4, k4, 10)
    with pytest.raises(ValueError):
        ring_swa.ring_sliding_window_attn(q4.float(), q4.float(), q4.float(), 10)


@pytest.mark.parametrize("path", sorted(glob.glob(os.path.join(GOLDEN, "ref_ring_d128_*.npz"))),
                         ids=lambda p: os.path.basename(p)[:-4])
def test_matches_reference_ring_vectors(path):
    """Global result of the reference's ring functions (their own code on gloo ranks) vs this
    implementation on one GPU, same bf16-representable inputs."""
    import ring_swa
    z = np.load(path)
    c = {k: z[k] for k in z.files}
    p = case_params(c)
    fn_name = str(c["fn"])
    varlen = "varlen" in fn_name
    q, k, v, do = make_inputs(p["seed"], p["T"], p["hq"], p["hkv"], p["d"], True, None if varlen else p["B"],
                              p["sink_rows"])
    kw = dict(window_size=p["W"])
    if varlen:
        kw.update(cu_seqlens=torch.tensor(p["cu"], dtype=torch.int32, device="cuda"), cp_size=1)
    out, dq, dk, dv = _run(getattr(ring_swa, fn_name), q.bfloat16(), k.bfloat16(), v.bfloat16(), do.bfloat16(), **kw)
    for n, a in (("out", out), ("dq", dq), ("dk", dk), ("dv", dv)):
        assert_close(n, a, torch.from_numpy(c[n].astype(np.float32)))


def _torch_block_reference(q, k, v, do, W, n_sink, a, b, heads):
    """fp32 torch attention on the token range [a - W, b + W) for a few heads, on the GPU: every query
    in [a, b + W) then has its complete window, so out/dq of queries [a, b) and dk/dv of keys [a, b)
    equal the full-sequence values (when n_sink == 0)."""
    lo, hi = max(0, a - W), min(q.shape[1], b + W)
    g = q.shape[2] // k.shape[2]
    kh = sorted({h // g for h in heads})
    assert len(kh) == 1
    qs = q[:, lo:hi, heads].float().requires_grad_(True)
    ks = k[:, lo:hi, kh].float().requires_grad_(True)
    vs = v[:, lo:hi, kh].float().requires_grad_(True)
    n = hi - lo
    i = torch.arange(n, device=q.device)
    mask = (i[None, :] <= i[:, None]) & (i[:, None] - i[None, :] <= W)
    s = torch.einsum("bihd,bjd->bhij", qs, ks[:, :, 0]) * (D ** -0.5)
    s = s.masked_fill(~mask, float("-inf"))
    lse = torch.logsumexp(s, -1)
    o = torch.einsum("bhij,bjd->bihd", torch.softmax(s, -1), vs[:, :, 0])
    o.backward(do[:, lo:hi, heads].float())
    sl = slice(a - lo, b - lo)
    return o.detach()[:, sl], lse[:, :, sl], qs.grad[:, sl], ks.grad[:, sl], vs.grad[:, sl]


def test_full_size_config_spot_blocks():
    """The headline configuration of the benchmark set at full size on one GPU (B=2, S=32768, 32/32 heads, W=1000): blocks of
    the result are compared with an fp32 torch computation of the same tokens, plus run-to-run
    agreement of the forward."""
    import ring_swa
    dev = torch.device("cuda")
    B, S, H, W = 2, 32768, 32, 1000
    g = torch.Generator(device=dev).manual_seed(1)
    q, k, v, do = (torch.randn(B, S, H, D, device=dev, generator=g).bfloat16() for _ in range(4))
    q.requires_grad_(True), k.requires_grad_(True), v.requires_grad_(True)
    out = ring_swa.ring_sliding_window_attn(q, k, v, W)
    out.backward(do)
    out2 = ring_swa.ring_sliding_window_attn(q.detach(), k.detach(), v.detach(), W)
    from ring_swa._kernels import check_device_status
    check_device_status()
    assert torch.equal(out, out2)
    for a, b, heads in ((0, 300, [0]), (5000, 5300, [7]), (32468, 32768, [31]), (16300, 16500, [16])):
        ro, _rl, rdq, rdk, rdv = _torch_block_reference(q.detach(), k.detach(), v.detach(), do, W, 0, a, b, heads)
        assert_close(f"out[{a}:{b}]", out.detach()[:, a:b, heads], ro)
        assert_close(f"dq[{a}:{b}]", q.grad[:, a:b, heads], rdq)
        assert_close(f"dk[{a}:{b}]", k.grad[:, a:b, heads], rdk)
        assert_close(f"dv[{a}:{b}]", v.grad[:, a:b, heads], rdv)


def _region_reference(q, k, v, do, W, n_sink, cu, a, b, q_heads):
    """fp32 torch attention, on the GPU, of the queries [a - 0, b + W) against the keys [a - W, b + W)
    (plus the sink tokens of the sequence, at their own positions), masked by the oracle's band_mask
    on GLOBAL positions.  out/dq of queries [a, b) and dk/dv of keys [a, b) then equal the values of
    the whole problem: every such query has its complete window, every such key all its queries.
    q_heads must be the query heads of ONE kv head.  Returns out, lse, dq (rows [a, b)), dk, dv (keys [a, b))."""
    from oracle.dense_attn import band_mask
    T = q.shape[1]
    g = q.shape[2] // k.shape[2]
    kh = q_heads[0] // g
    assert all(h // g == kh for h in q_heads)
    lo, hi = max(0, a - W), min(T, b + W)
    q_pos = torch.arange(a, hi)
    key_idx = torch.arange(lo, hi)
    if n_sink:
        starts = [0] if cu is None else cu[:-1]
        s0 = max(s for s in starts if s <= a)
        sink = torch.arange(s0, min(s0 + n_sink, lo))       # sink tokens that lie outside the window range
        key_idx = torch.cat([sink, key_idx])
    mask = band_mask(q_pos, key_idx, W, n_sink, cu).to(q.device)
    dev_idx = key_idx.to(q.device)
    qs = q[:, a:hi, q_heads].float().requires_grad_(True)
    ks = k[:, dev_idx][:, :, kh].float().requires_grad_(True)
    vs = v[:, dev_idx][:, :, kh].float().requires_grad_(True)
    s = torch.einsum("bihd,bjd->bhij", qs, ks) * (D ** -0.5)
    s = s.masked_fill(~mask[None, None], float("-inf"))
    lse = torch.logsumexp(s, -1)
    o = torch.einsum("bhij,bjd->bihd", torch.softmax(s, -1), vs)
    o.backward(do[:, a:hi, q_heads].float())
    n_lead = key_idx.numel() - (hi - lo)                    # sink rows in front
    ksl = slice(n_lead + a - lo, n_lead + b - lo)
    return o.detach()[:, : b - a], lse[:, :, : b - a], qs.grad[:, : b - a], ks.grad[:, ksl], vs.grad[:, ksl]


@pytest.mark.parametrize("name", ["cfg3", "cfg4"])
def test_full_size_varlen_and_sink_spot_blocks(name):
    """The packed configuration (7 sequences, 32/8 heads, W=4096, 65536 tokens) and the sink + window one
    (32/8 heads, W=8192, 131072 tokens) of the benchmark set at full size on one GPU: blocks of out, dq, dk, dv against fp32 torch
    on the same tokens; the backward is deterministic, so a second run must agree bit for bit."""
    import ring_swa
    dev = torch.device("cuda")
    Hq, Hkv = 32, 8
    if name == "cfg3":
        lens = [7204, 3978, 14070, 10318, 13142, 12634, 4190]
        cu = [0]
        for L in lens:
            cu.append(cu[-1] + L)
        T, W, n_sink, seed = 65536, 4096, 0, 2
        blocks = [(7100, 7300, [4, 5, 6, 7]), (30000, 30160, [28, 29, 30, 31]), (65400, 65536, [0, 1, 2, 3])]
    else:
        cu = None
        T, W, n_sink, seed = 131072, 8192, 1, 3
        blocks = [(0, 128, [0, 1, 2, 3]), (50000, 50128, [12, 13, 14, 15]), (130944, 131072, [28, 29, 30, 31])]
    g = torch.Generator(device=dev).manual_seed(seed)
    q, k, v, do = (torch.randn(1, T, h, D, device=dev, generator=g).bfloat16() for h in (Hq, Hkv, Hkv, Hq))

    def run():
        qq, kk, vv = (t.detach().clone().requires_grad_(True) for t in (q, k, v))
        if name == "cfg3":
            out = ring_swa.ring_sliding_window_attn_varlen(
                qq[0], kk[0], vv[0], W, torch.tensor(cu, dtype=torch.int32, device=dev), cp_size=1)[None]
        else:
            out = ring_swa.ring_streaming_llm_attn(qq, kk, vv, W)
        out.backward(do)
        return out.detach(), qq.grad, kk.grad, vv.grad

    got = run()
    again = run()
    from ring_swa._kernels import check_device_status
    check_device_status()
    for x, y in zip(got, again):
        assert torch.equal(x, y)
    out, dq, dk, dv = got
    for a, b, heads in blocks:
        ro, _rl, rdq, rdk, rdv = _region_reference(q, k, v, do, W, n_sink, cu, a, b, heads)
        kh = [heads[0] // (Hq // Hkv)]
        assert_close(f"out[{a}:{b}]", out[:, a:b, heads], ro)
        assert_close(f"dq[{a}:{b}]", dq[:, a:b, heads], rdq)
        lo_k = max(a, n_sink) if a == 0 else a           # the sink key's own gradient gathers every later query
        sl = slice(lo_k - a, b - a)
        assert_close(f"dk[{lo_k}:{b}]", dk[:, lo_k:b, kh][:, :, 0], rdk[:, sl])
        assert_close(f"dv[{lo_k}:{b}]", dv[:, lo_k:b, kh][:, :, 0], rdv[:, sl])
        torch.cuda.empty_cache()


def _chunked_block_reference(q, k, v, do, W, a, b, kh, q_chunk=2048):
    """fp32 torch reference, on the GPU, for plain sliding-window attention at sizes where the scores of a
    whole block's window no longer fit at once: out, lse, dq of queries [a, b) and dk, dv of keys [a, b) of
    KV head kh (summed over its query heads), from explicit formulas, query chunk by query chunk.  Every
    query that sees a key of [a, b) -- positions [a, b + W] -- is walked with its complete window."""
    T, Hq, Hkv = q.shape[1], q.shape[2], k.shape[2]
    g = Hq // Hkv
    heads = list(range(kh * g, kh * g + g))
    scale = D ** -0.5
    dk = torch.zeros(b - a, D, dtype=torch.float32, device=q.device)
    dv = torch.zeros_like(dk)
    out_b = lse_b = dq_b = None
    hi = min(T, b + W + 1)
    for c0 in range(a, hi, q_chunk):
        c1 = min(hi, c0 + q_chunk)
        k0 = max(0, c0 - W)
        qs = q[0, c0:c1, heads].float()                      # [n, g, D]
        dos = do[0, c0:c1, heads].float()
        ks, vs = k[0, k0:c1, kh].float(), v[0, k0:c1, kh].float()   # [m, D]
        pq = torch.arange(c0, c1, device=q.device)[:, None]
        pk = torch.arange(k0, c1, device=q.device)[None, :]
        mask = (pk <= pq) & (pq - pk <= W)
        s = torch.einsum("nhd,md->hnm", qs, ks) * scale
        s = s.masked_fill(~mask[None], float("-inf"))
        lse = torch.logsumexp(s, -1)                         # [g, n]
        p = torch.exp(s - lse[..., None])
        o = torch.einsum("hnm,md->nhd", p, vs)
        delta = (o * dos).sum(-1).transpose(0, 1)            # [g, n]
        dp = torch.einsum("nhd,md->hnm", dos, vs)
        ds = p * (dp - delta[..., None])
        if c0 == a:                                          # the block's own queries are the chunk's first rows
            n = b - a
            out_b, lse_b = o[:n], lse[:, :n]
            dq_b = torch.einsum("hnm,md->nhd", ds[:, :n], ks) * scale
        lo_k, hi_k = max(a, k0), min(b, c1)                  # keys of [a, b) this chunk holds
        if lo_k < hi_k:
            sl = slice(lo_k - k0, hi_k - k0)
            dv[lo_k - a:hi_k - a] += torch.einsum("hnm,nhd->md", p[:, :, sl], dos)
            dk[lo_k - a:hi_k - a] += torch.einsum("hnm,nhd->md", ds[:, :, sl], qs) * scale
        del s, p, dp, ds
    return out_b, lse_b, dq_b, dk, dv, heads


@pytest.mark.timeout(900)
def test_full_size_long_window_spot_blocks():
    """The multi-hop configuration of the benchmark set at full size on one GPU (B=1, S=262144, 64/8 heads,
    W=65536): a query tile there accumulates over up to 513 key tiles and a key tile's gradients over 8 heads
    times 513 query tiles.  Blocks of out, dq, dk, dv against fp32 torch on the same tokens, and run-to-run
    bit equality."""
    import ring_swa
    dev = torch.device("cuda")
    T, Hq, Hkv, W = 262144, 64, 8, 65536
    g = torch.Generator(device=dev).manual_seed(4)
    q, k, v, do = (torch.randn(1, T, h, D, device=dev, generator=g).bfloat16() for h in (Hq, Hkv, Hkv, Hq))

    def run():
        qq, kk, vv = (t.detach().clone().requires_grad_(True) for t in (q, k, v))
        out = ring_swa.ring_sliding_window_attn(qq, kk, vv, W)
        out.backward(do)
        return out.detach(), qq.grad, kk.grad, vv.grad

    got = run()
    again = run()
    from ring_swa._kernels import check_device_status
    check_device_status()
    for x, y in zip(got, again):
        assert torch.equal(x, y)
    del again
    out, dq, dk, dv = got
    for a, kh in ((0, 0), (131072 - 64, 3), (T - 128, 7)):
        b = a + 128
        ro, _rl, rdq, rdk, rdv, heads = _chunked_block_reference(q, k, v, do, W, a, b, kh)
        assert_close(f"out[{a}:{b}]", out[0, a:b, heads], ro)
        assert_close(f"dq[{a}:{b}]", dq[0, a:b, heads], rdq)
        assert_close(f"dk[{a}:{b}]", dk[0, a:b, kh], rdk)
        assert_close(f"dv[{a}:{b}]", dv[0, a:b, kh], rdv)
        torch.cuda.empty_cache()
