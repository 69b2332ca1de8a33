"""CUDA kernels against the CPU oracle, called through the C ABI (ring_swa._kernels -> librswa.so)."""
import pytest
import torch

from gpu_util import assert_close, assert_lse_close, randn_bf16
from oracle.dense_attn import dense_attn, dense_attn_fwd_bwd, merge_partials

pytestmark = pytest.mark.gpu

D = 128


def _K():
    from ring_swa import _kernels
    return _kernels


def _cu(lens):
    cu = [0]
    for L in lens:
        cu.append(cu[-1] + L)
    return cu


@pytest.mark.parametrize("mode", [0, 1, 2, 3])
def test_tensor_core_operand_paths(mode):
    K = _K()
    dev = torch.device("cuda")
    a = randn_bf16(128, 128, seed=1).to(dev)
    b = randn_bf16(128, 128, seed=2).to(dev)
    af, bf = a.float(), b.float()
    ref = [af @ bf.T, af @ bf, af @ bf, af.T @ bf][mode]
    d = K.selftest_mma(mode, a, b)
    K.check_device_status()
    assert (d - ref).abs().max().item() < 1e-3


CASES = [
    # name, B, S, Hq, Hkv, W, n_sink, lens
    ("one_tile", 1, 128, 1, 1, 1000, 0, None),
    ("tiny", 1, 5, 2, 1, 2, 0, None),
    ("w0", 1, 200, 2, 2, 0, 0, None),
    ("band", 1, 512, 2, 2, 100, 0, None),
    ("band_tile_edges", 1, 640, 2, 1, 127, 0, None),
    ("band_tile_edges2", 1, 640, 2, 1, 128, 0, None),
    ("band_tile_edges3", 1, 640, 2, 1, 129, 0, None),
    ("ragged_batch", 2, 300, 4, 2, 77, 0, None),
    ("gqa8", 1, 384, 8, 1, 200, 0, None),
    ("full_causal", 1, 700, 2, 2, 100000, 0, None),
    ("sink1", 1, 640, 4, 1, 130, 1, None),
    ("sink4", 1, 640, 2, 1, 130, 4, None),
    ("sink_big_window", 1, 300, 2, 1, 1000, 1, None),
    ("sink_batch", 2, 520, 2, 2, 64, 1, None),
    ("varlen", 1, 700, 4, 2, 150, 0, [100, 1, 299, 300]),
    ("varlen_tiny_seqs", 1, 300, 2, 1, 10, 0, [1, 1, 2, 127, 1, 128, 40]),
    ("varlen_sink", 1, 700, 4, 2, 90, 1, [100, 1, 299, 300]),
    ("varlen_sink3", 1, 900, 2, 1, 40, 3, [2, 1, 400, 497]),
    ("varlen_tile_aligned", 1, 512, 2, 2, 200, 1, [128, 128, 256]),
]


@pytest.mark.parametrize("name,B,S,Hq,Hkv,W,n_sink,lens", CASES, ids=[c[0] for c in CASES])
def test_fwd_bwd_matches_oracle(name, B, S, Hq, Hkv, W, n_sink, lens):
    K = _K()
    dev = torch.device("cuda")
    q = randn_bf16(B, S, Hq, D, seed=10)
    k = randn_bf16(B, S, Hkv, D, seed=11)
    v = randn_bf16(B, S, Hkv, D, seed=12)
    do = randn_bf16(B, S, Hq, D, seed=13)
    cu = _cu(lens) if lens else None
    scale = D ** -0.5
    ro, rl, rdq, rdk, rdv = dense_attn_fwd_bwd(q, k, v, do, W, scale, n_sink, cu)
    qd, kd, vd, dod = (x.to(dev) for x in (q, k, v, do))
    cud = torch.tensor(cu, dtype=torch.int32, device=dev) if cu else None
    out, lse = K.fwd(qd, [K.KVSpan(kd, vd, 0)], W, n_sink, scale, 0, cud)
    K.check_device_status()
    assert_close("out", out, ro)
    assert_lse_close(lse, rl)
    dq, dk, dv = torch.empty_like(qd), torch.empty_like(kd), torch.empty_like(vd)
    K.bwd(qd, [K.KVSpan(kd, vd, 0, dk=dk, dv=dv)], out, lse, dod, dq, W, n_sink, scale, 0, cud)
    K.check_device_status()
    assert_close("dq", dq, rdq)
    assert_close("dk", dk, rdk)
    assert_close("dv", dv, rdv)


def test_fp16_and_fp32_grads_and_strided_inputs():
    K = _K()
    dev = torch.device("cuda")
    B, S, Hq, Hkv, W = 1, 400, 4, 2, 90
    g = torch.Generator().manual_seed(5)
    qkv = torch.randn(B, S, Hq + 2 * Hkv, D, generator=g).half()     # packed projection output
    do = torch.randn(B, S, Hq, D, generator=g).half()
    q, k, v = qkv[:, :, :Hq], qkv[:, :, Hq:Hq + Hkv], qkv[:, :, Hq + Hkv:]
    ro, rl, rdq, rdk, rdv = dense_attn_fwd_bwd(q, k, v, do, W, None, 0, None)
    qkvd = qkv.to(dev)
    qd, kd, vd = qkvd[:, :, :Hq], qkvd[:, :, Hq:Hq + Hkv], qkvd[:, :, Hq + Hkv:]
    out, lse = K.fwd(qd, [K.KVSpan(kd, vd, 0)], W, 0, D ** -0.5)
    assert_close("out", out, ro)
    assert_lse_close(lse, rl)
    dq = torch.empty_like(out)
    dk = torch.empty(B, S, Hkv, D, dtype=torch.float32, device=dev)
    dv = torch.empty_like(dk)
    K.bwd(qd, [K.KVSpan(kd, vd, 0, dk=dk, dv=dv)], out, lse, do.to(dev), dq, W, 0, D ** -0.5)
    K.check_device_status()
    assert_close("dq", dq, rdq)
    assert_close("dk", dk, rdk)
    assert_close("dv", dv, rdv)


@pytest.mark.parametrize("cp,S,W,n_sink,lens", [
    (2, 192, 100, 0, None),
    (4, 128, 300, 0, None),          # window spans two earlier ranks
    (3, 200, 64, 1, None),           # sink fetched from rank 0
    (4, 128, 200, 4, None),
    (2, 192, 90, 0, [100, 1, 155, 128]),
    (4, 128, 140, 1, [290, 222]),
    (4, 128, 50, 2, [130, 200, 182]),
    (4, 128, 40, 3, [127, 128, 257]),    # sink tokens of a sequence lie on two ranks (127 | 128, 129)
    (3, 200, 30, 5, [398, 202]),         # ... 398, 399 on rank 1 and 400-402 on rank 2, needed by nobody later
    (4, 128, 20, 4, [254, 258]),         # sinks 254, 255 | 256, 257: rank 3 needs both pieces
])
def test_spans_emulated_ranks(cp, S, W, n_sink, lens):
    """Every rank's forward/backward over (sink | halo... | local) spans, run one after the other on
    one GPU, reproduces the global result; halo gradients are added on the owner as the ring does."""
    from ring_swa._plan import make_plan
    K = _K()
    dev = torch.device("cuda")
    T, Hq, Hkv = cp * S, 4, 2
    q = randn_bf16(1, T, Hq, D, seed=20)
    k = randn_bf16(1, T, Hkv, D, seed=21)
    v = randn_bf16(1, T, Hkv, D, seed=22)
    do = randn_bf16(1, T, Hq, D, seed=23)
    cu = _cu(lens) if lens else None
    scale = D ** -0.5
    ro, rl, rdq, rdk, rdv = dense_attn_fwd_bwd(q, k, v, do, W, scale, n_sink, cu)
    qd, kd, vd, dod = (x.to(dev) for x in (q, k, v, do))
    cud = torch.tensor(cu, dtype=torch.int32, device=dev) if cu else None
    dk_acc = torch.zeros(1, T, Hkv, D, dtype=torch.float32, device=dev)
    dv_acc = torch.zeros_like(dk_acc)
    for r in range(cp):
        plan = make_plan(cp, r, S, W, n_sink, cu)
        sl = slice(r * S, (r + 1) * S)
        spans, ranges = [], []
        for sr in plan.sink_recv:
            ranges.append((sr.pos_start, sr.pos_start + sr.n))
        for h in plan.halo_recv[::-1]:
            ranges.append((h.pos_start, h.pos_start + h.length))
        ranges.append((r * S, (r + 1) * S))
        for a, b in ranges:
            kk, vv = kd[:, a:b].contiguous(), vd[:, a:b].contiguous()
            spans.append(K.KVSpan(kk, vv, a, dk=torch.empty(kk.shape, dtype=torch.float32, device=dev),
                                  dv=torch.empty(kk.shape, dtype=torch.float32, device=dev)))
        out, lse = K.fwd(qd[:, sl], spans, W, n_sink, scale, r * S, cud)
        K.check_device_status()
        assert_close(f"out[rank {r}]", out, ro[:, sl])
        assert_lse_close(lse, rl[:, :, sl])
        dq = torch.empty_like(out)
        K.bwd(qd[:, sl], spans, out, lse, dod[:, sl], dq, W, n_sink, scale, r * S, cud)
        K.check_device_status()
        assert_close(f"dq[rank {r}]", dq, rdq[:, sl])
        for (a, b), sp in zip(ranges, spans):
            dk_acc[:, a:b] += sp.dk
            dv_acc[:, a:b] += sp.dv
    assert_close("dk", dk_acc, rdk)
    assert_close("dv", dv_acc, rdv)


def test_two_phase_forward_and_split_backward():
    """Query-tile ranges, the (local | halo) partials + merge path and a backward split over two calls."""
    from ring_swa import _C
    K = _K()
    dev = torch.device("cuda")
    S, Hq, Hkv, W = 384, 4, 2, 500
    q = randn_bf16(1, S, Hq, D, seed=30).to(dev)
    kh = randn_bf16(1, 300, Hkv, D, seed=31).to(dev)
    vh = randn_bf16(1, 300, Hkv, D, seed=32).to(dev)
    kl = randn_bf16(1, S, Hkv, D, seed=33).to(dev)
    vl = randn_bf16(1, S, Hkv, D, seed=34).to(dev)
    do = randn_bf16(1, S, Hq, D, seed=35).to(dev)
    scale = D ** -0.5
    kall, vall = torch.cat([kh, kl], 1).cpu(), torch.cat([vh, vl], 1).cpu()
    qf = q.cpu().float().requires_grad_(True)
    kf, vf = kall.float().requires_grad_(True), vall.float().requires_grad_(True)
    ro, rl = dense_attn(qf, kf, vf, W, scale, 0, None, q_pos0=300, k_pos0=0)
    ro.backward(do.cpu().float())
    halo, local = K.KVSpan(kh, vh, 0), K.KVSpan(kl, vl, 300)
    # (a) tile ranges: tiles [1,3) then [0,1)
    out = torch.zeros_like(q)
    lse = torch.zeros(1, Hq, S, dtype=torch.float32, device=dev)
    K.fwd(q, [halo, local], W, 0, scale, 300, out=out, lse=lse, q_tiles=(1, 3))
    K.fwd(q, [halo, local], W, 0, scale, 300, out=out, lse=lse, q_tiles=(0, 1))
    assert_close("out(tile ranges)", out, ro)
    assert_lse_close(lse, rl)
    # (b) partials + merge
    o1, l1 = K.fwd(q, [local], W, 0, scale, 300)
    o2, l2 = K.fwd(q, [halo], W, 0, scale, 300)
    K.merge(o1, l1, o2, l2)
    assert_close("out(merge)", o1, ro)
    assert_lse_close(l1, rl)
    # (b') the halo pass continues the local partial result inside the kernel, in place
    o3, l3 = K.fwd(q, [local], W, 0, scale, 300)
    K.fwd(q, [halo], W, 0, scale, 300, out=o3, lse=l3, carry=True)
    assert_close("out(carried)", o3, ro)
    assert_lse_close(l3, rl)
    # ... and the other way round: the halo first (rows beyond its reach start empty, lse = -inf), then
    # the local keys carried on top; rows that see nothing of the second call keep what they hold
    o4, l4 = K.fwd(q, [halo], W, 0, scale, 300)
    K.fwd(q, [local], W, 0, scale, 300, out=o4, lse=l4, carry=True)
    assert_close("out(carried, halo first)", o4, ro)
    assert_lse_close(l4, rl)
    o5, l5 = o4.clone(), l4.clone()
    far = K.KVSpan(kh, vh, 100000)          # keys no query of this call can see
    K.fwd(q, [far], W, 0, scale, 300, out=o5, lse=l5, carry=True)
    assert torch.equal(o5, o4) and torch.equal(l5, l4)
    # (c) backward in two calls sharing the workspace
    dq = torch.empty_like(q)
    halo.dk, halo.dv = torch.empty_like(kh), torch.empty_like(vh)
    local.dk, local.dv = torch.empty_like(kl), torch.empty_like(vl)
    ws = K.bwd(q, [halo], out, lse, do, dq, W, 0, scale, 300, flags=_C.BWD_INIT)
    seen = K.KVSpan(kh, vh, 0)      # second call: no gradient buffers for the halo, dq over both spans
    K.bwd(q, [seen, local], out, lse, do, dq, W, 0, scale, 300, workspace=ws, flags=_C.BWD_FINISH)
    K.check_device_status()
    assert_close("dq", dq, qf.grad)
    assert_close("dk", torch.cat([halo.dk, local.dk], 1), kf.grad)
    assert_close("dv", torch.cat([halo.dv, local.dv], 1), vf.grad)


def test_empty_visibility_gives_zero_and_minus_inf():
    K = _K()
    dev = torch.device("cuda")
    q = randn_bf16(1, 256, 2, D, seed=40).to(dev)
    k = randn_bf16(1, 64, 2, D, seed=41).to(dev)
    v = randn_bf16(1, 64, 2, D, seed=42).to(dev)
    # keys at positions [0, 64), queries at [1000, 1256), window 100: nothing visible
    out, lse = K.fwd(q, [K.KVSpan(k, v, 0)], 100, 0, 0.1, 1000)
    K.check_device_status()
    assert (out == 0).all() and torch.isinf(lse).all() and (lse < 0).all()
    o2, l2 = K.fwd(q, [K.KVSpan(k, v, 0)], 100, 0, 0.1, 1000)
    K.merge(out, lse, o2, l2)
    assert (out == 0).all() and torch.isinf(lse).all()


def test_merge_halo_accumulate_cast():
    K = _K()
    dev = torch.device("cuda")
    B, S, H = 2, 333, 3
    oa, ob = randn_bf16(B, S, H, D, seed=50), randn_bf16(B, S, H, D, seed=51)
    g = torch.Generator().manual_seed(52)
    la, lb = torch.randn(B, H, S, generator=g) * 3, torch.randn(B, H, S, generator=g) * 3
    la[0, 0, :5] = float("-inf")
    lb[0, 1, :5] = float("-inf")
    ro, rl = merge_partials(oa.float(), la, ob.float(), lb)
    oad, lad = oa.to(dev), la.to(dev)
    K.merge(oad, lad, ob.to(dev), lb.to(dev))
    assert_close("merge out", oad, ro, atol=1e-2)
    assert_lse_close(lad, rl, tol=1e-5)
    acc = torch.randn(2, 100, 2, D, generator=g)
    recv = torch.randn(2, 40, 2, D, generator=g).bfloat16()
    accd = acc.to(dev)
    K.halo_accumulate(accd[:, 60:], recv.to(dev))
    ref = acc.clone()
    ref[:, 60:] += recv.float()
    assert torch.equal(accd.cpu(), ref)
    recv32 = torch.randn(2, 40, 2, D, generator=g)
    K.halo_accumulate(accd[:, :40], recv32.to(dev))
    ref[:, :40] += recv32
    assert torch.equal(accd.cpu(), ref)
    dst = torch.empty(2, 100, 2, D, dtype=torch.bfloat16, device=dev)
    K.cast_from_f32(dst, accd)
    assert torch.equal(dst.cpu(), ref.bfloat16())


def test_argument_errors_are_raised_not_faulted():
    K = _K()
    dev = torch.device("cuda")
    q = torch.zeros(1, 128, 2, 64, dtype=torch.bfloat16, device=dev)
    with pytest.raises(ValueError):
        K.fwd(q, [K.KVSpan(q, q, 0)], 10, 0, 0.1)
    q = torch.zeros(1, 128, 3, D, dtype=torch.bfloat16, device=dev)
    k = torch.zeros(1, 128, 2, D, dtype=torch.bfloat16, device=dev)
    with pytest.raises(ValueError, match="divisible"):
        K.fwd(q, [K.KVSpan(k, k, 0)], 10, 0, 0.1)
    with pytest.raises(ValueError, match="overlap"):
        K.fwd(k, [K.KVSpan(k, k, 0), K.KVSpan(k, k, 100)], 10, 0, 0.1)
    with pytest.raises(ValueError):
        K.fwd(k.float(), [K.KVSpan(k, k, 0)], 10, 0, 0.1)
    with pytest.raises(RuntimeError, match="no CPU path"):
        K.fwd(k.cpu(), [K.KVSpan(k.cpu(), k.cpu(), 0)], 10, 0, 0.1)


def test_backward_called_first_from_a_fresh_thread():
    """The autograd engine calls the backward from a worker thread that may not have made any CUDA call
    of its own yet; building the tensor maps there must still work (the library binds a context itself)."""
    import threading
    K = _K()
    dev = torch.device("cuda")
    B, S, H, W = 1, 256, 2, 100
    q, k, v, do = (randn_bf16(B, S, H, D, seed=70 + i).to(dev) for i in range(4))
    out, lse = K.fwd(q, [K.KVSpan(k, v, 0)], W, 0, D ** -0.5)
    ref = [torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)]
    K.bwd(q, [K.KVSpan(k, v, 0, dk=ref[1], dv=ref[2])], out, lse, do, ref[0], W, 0, D ** -0.5)
    got = [torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)]
    ws = K.bwd_workspace(q)
    stream = torch.cuda.current_stream()
    err = []

    def run():
        try:
            with torch.cuda.stream(stream):
                K.bwd(q, [K.KVSpan(k, v, 0, dk=got[1], dv=got[2])], out, lse, do, got[0], W, 0, D ** -0.5, workspace=ws)
        except Exception as e:  # noqa: BLE001 - reported below
            err.append(e)

    th = threading.Thread(target=run)
    th.start()
    th.join()
    assert not err, err
    torch.cuda.synchronize()
    for a, b in zip(got, ref):
        assert torch.equal(a, b)      # the backward is deterministic


def test_peer_put_and_bounded_flag_wait():
    """The pieces of the peer-store exchange on one GPU (destination and flag in local memory): a strided
    source lands densely and the flag carries its number; a wait for a number that nobody writes gives up
    after its limit and reports through the status word, leaving the context usable."""
    K = _K()
    dev = torch.device("cuda")
    big = torch.arange(4 * 3000, dtype=torch.float32, device=dev).reshape(4, 3000)
    src = big[:, 1000:2000]                      # rows of 1000 floats, 3000 apart
    dst = torch.zeros(4, 1000, dtype=torch.float32, device=dev)
    flags = torch.zeros(8, dtype=torch.int32, device=dev)
    K.peer_put(dst.data_ptr(), 4000, src, flags.data_ptr(), 7)
    K.flag_wait(flags.data_ptr(), 7, dev, timeout_s=2.0)
    after = dst.clone()                          # launched behind the wait: sees the data
    torch.cuda.synchronize()
    assert torch.equal(after, src) and int(flags[0]) == 7
    K.check_device_status()
    K.flag_wait(flags.data_ptr(), 5, dev, timeout_s=2.0)      # numbers only grow: an older one is reached already
    K.check_device_status()
    K.flag_wait(flags[1:].data_ptr(), 1, dev, timeout_s=0.02)   # nobody writes this word
    with pytest.raises(RuntimeError, match="device-side error code 105"):
        K.check_device_status()
    K.flag_set(flags[1:].data_ptr(), 1)
    K.flag_wait(flags[1:].data_ptr(), 1, dev, timeout_s=2.0)
    K.check_device_status()
