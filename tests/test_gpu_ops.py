"""The operator-level functions of ring_swa.ops (the names the reference binds flash-attn and its Triton
merge under) against the dense float32 restatement of flash-attn's band, on the GPU through librswa.so."""
import pytest
import torch

from flash_band import attn, attn_fwd_bwd
from gpu_util import assert_close, assert_lse_close, randn_bf16

pytestmark = pytest.mark.gpu

D = 128
SCALE = D ** -0.5


def _dev():
    return torch.device("cuda")


CASES = [
    # Sq, Sk, Hq, Hkv, window, causal
    (200, 200, 2, 2, (50, 0), True),        # the diagonal call of the ring
    (200, 200, 4, 2, (50, 50), False),      # the shape the reference's own flash test uses (test/test_local_swa.py:98-144)
    (130, 300, 2, 1, (64, 0), True),        # fewer queries than keys, bottom-right aligned
    (300, 130, 2, 2, (40, 0), True),        # more queries than keys: leading rows see nothing
    (257, 257, 2, 2, (-1, -1), False),      # full attention
    (128, 256, 2, 2, (0, 128), False),      # off-diagonal hop with W = k*S (keys b >= a)
    (192, 192, 2, 2, (-1, 0), True),        # plain causal
    (150, 150, 2, 2, (20, 70), False),
]


@pytest.mark.parametrize("Sq,Sk,Hq,Hkv,window,causal", CASES)
def test_wrapped_flash_attn_fwd_bwd(Sq, Sk, Hq, Hkv, window, causal):
    from ring_swa.ops import wrapped_flash_attn_bwd, wrapped_flash_attn_fwd
    B = 2
    q, k, v, do = (randn_bf16(B, s, h, D, seed=i) for i, (s, h) in enumerate([(Sq, Hq), (Sk, Hkv), (Sk, Hkv), (Sq, Hq)]))
    ro, rl, rdq, rdk, rdv = attn_fwd_bwd(q, k, v, do, SCALE, window, causal)
    qd, kd, vd, dod = (t.to(_dev()) for t in (q, k, v, do))
    out, lse = wrapped_flash_attn_fwd(qd, kd, vd, SCALE, window, causal)
    assert out.dtype == torch.bfloat16 and lse.dtype == torch.float32 and lse.shape == (B, Hq, Sq)
    assert_close("out", out, ro)
    assert_lse_close(lse, rl)
    dq = torch.empty_like(qd)
    dkv = torch.empty(2, B, Sk, Hkv, D, dtype=torch.bfloat16, device=_dev())
    wrapped_flash_attn_bwd(qd, kd, vd, out, lse, dod, dq, dkv[0], dkv[1], SCALE, window, causal)
    assert_close("dq", dq, rdq)
    assert_close("dk", dkv[0], rdk)
    assert_close("dv", dkv[1], rdv)
    from ring_swa import _kernels
    _kernels.check_device_status()


def _packed_reference(q, k, v, do, cu_q, cu_k, window, causal):
    outs, lses, dqs, dks, dvs = [], [], [], [], []
    for i in range(len(cu_q) - 1):
        a, b, c, d = cu_q[i], cu_q[i + 1], cu_k[i], cu_k[i + 1]
        o, l, gq, gk, gv = attn_fwd_bwd(q[None, a:b], k[None, c:d], v[None, c:d], do[None, a:b], SCALE, window, causal)
        outs.append(o[0]); lses.append(l[0]); dqs.append(gq[0]); dks.append(gk[0]); dvs.append(gv[0])
    return torch.cat(outs), torch.cat(lses, dim=1), torch.cat(dqs), torch.cat(dks), torch.cat(dvs)


@pytest.mark.parametrize("lens_q,lens_k,window,causal", [
    ([100, 37, 250, 13], None, (60, 0), True),                    # one set of boundaries: single launch
    ([100, 37, 250], [100, 37, 250], (30, 20), False),            # same lengths, looks right: per sequence
    ([64, 130, 9], [200, 130, 40], (50, 0), True),                # different query / key lengths
    ([150], [90], (45, 0), False),                                # the rectangular off-diagonal call (ring_swa/sliding_window/varlen.py:147-169)
])
def test_wrapped_flash_attn_varlen(lens_q, lens_k, window, causal):
    from ring_swa.ops import wrapped_flash_attn_bwd_varlen, wrapped_flash_attn_fwd_varlen
    Hq, Hkv = 4, 2
    cu_q = [0]
    for L in lens_q:
        cu_q.append(cu_q[-1] + L)
    cu_k = cu_q if lens_k is None else [0]
    if lens_k is not None:
        for L in lens_k:
            cu_k.append(cu_k[-1] + L)
    Tq, Tk = cu_q[-1], cu_k[-1]
    q, do = randn_bf16(Tq, Hq, D, seed=11), randn_bf16(Tq, Hq, D, seed=14)
    k, v = randn_bf16(Tk, Hkv, D, seed=12), randn_bf16(Tk, Hkv, D, seed=13)
    ro, rl, rdq, rdk, rdv = _packed_reference(q, k, v, do, cu_q, cu_k, window, causal)
    dev = _dev()
    cq = torch.tensor(cu_q, dtype=torch.int32, device=dev)
    ck = cq if lens_k is None else torch.tensor(cu_k, dtype=torch.int32, device=dev)
    qd, kd, vd, dod = (t.to(dev) for t in (q, k, v, do))
    out, lse = wrapped_flash_attn_fwd_varlen(qd, kd, vd, SCALE, window, cq, ck, max(lens_q), max(lens_k or lens_q), causal)
    assert out.shape == (Tq, Hq, D) and lse.shape == (Hq, Tq)
    assert_close("out", out, ro)
    assert_lse_close(lse, rl)
    dq, dk, dv = torch.empty_like(qd), torch.empty_like(kd), torch.empty_like(vd)
    wrapped_flash_attn_bwd_varlen(qd, kd, vd, out, lse, dod, dq, dk, dv, SCALE, window, cq, ck,
                                  max(lens_q), max(lens_k or lens_q), causal)
    assert_close("dq", dq, rdq)
    assert_close("dk", dk, rdk)
    assert_close("dv", dv, rdv)


def _torch_merge(acc, lse, new, new_lse):
    """The reference's torch formula (ring_swa/ops/merge.py:16-50) in float64, -inf pairs giving (0, -inf)."""
    lse, new_lse = lse.double(), new_lse.double()
    mx = torch.maximum(lse, new_lse)
    both = torch.isinf(mx) & (mx < 0)
    safe = torch.where(both, torch.zeros_like(mx), mx)
    wa, wb = torch.exp(lse - safe), torch.exp(new_lse - safe)
    tot = torch.where(both, torch.ones_like(wa), wa + wb)
    out = acc.double() * (wa / tot).movedim(1, 2)[..., None] + new.double() * (wb / tot).movedim(1, 2)[..., None]
    out = torch.where(both.movedim(1, 2)[..., None], torch.zeros_like(out), out)
    return out, torch.where(both, mx, safe + torch.log(tot))


@pytest.mark.parametrize("lse_dtype", [torch.float32, torch.float64])
@pytest.mark.parametrize("new_dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_merge_attn_out_reference_accumulators(lse_dtype, new_dtype):
    """float32 output / float64 lse accumulators, as the reference's ring loop keeps them."""
    from ring_swa.ops import merge_attn_out
    B, S, H, Dm = 2, 77, 3, 64
    g = torch.Generator().manual_seed(5)
    acc = torch.randn(B, S + 10, H, Dm, generator=g)
    new = torch.randn(B, S, H, Dm, generator=g).to(new_dtype)
    lse = (torch.randn(B, H, S + 10, generator=g) * 3).to(lse_dtype)
    new_lse = torch.randn(B, H, S, generator=g) * 3
    lse[0, 0, :4] = float("-inf")                 # nothing accumulated yet: the new partial is taken as is
    new_lse[1, 2, 5:9] = float("-inf")
    lse[1, 1, 20] = new_lse[1, 1, 10] = float("-inf")
    ro, rl = _torch_merge(acc[:, 10:], lse[:, :, 10:], new.float(), new_lse)
    dev = _dev()
    accd, lsed = acc.to(dev), lse.to(dev)
    merge_attn_out(accd[:, 10:], lsed[:, :, 10:], new.to(dev), new_lse.to(dev))     # strided views, in place
    assert torch.equal(accd[:, :10].cpu(), acc[:, :10]) and torch.equal(lsed[:, :, :10].cpu(), lse[:, :, :10])
    assert_close("merged out", accd[:, 10:], ro.float(), atol=1e-5, rtol=1e-5, rel_l2=1e-5)
    assert_lse_close(lsed[:, :, 10:], rl.float(), tol=1e-5)
    assert lsed.dtype == lse_dtype


def test_flash_attn_funcs_accumulate_like_the_reference_loop():
    """Two partial results over disjoint key blocks merged through flash_attn_fwd_func equal attention
    over all keys; flash_attn_bwd_func with the final out / lse gives each block's gradients."""
    from ring_swa.ops import flash_attn_bwd_func, flash_attn_fwd_func
    B, S, Hq, Hkv, W = 1, 256, 2, 2, 300
    dev = _dev()
    q, do = randn_bf16(B, S, Hq, D, seed=31), randn_bf16(B, S, Hq, D, seed=34)
    kv_prev = torch.stack([randn_bf16(B, S, Hkv, D, seed=32), randn_bf16(B, S, Hkv, D, seed=33)])
    kv_own = torch.stack([randn_bf16(B, S, Hkv, D, seed=35), randn_bf16(B, S, Hkv, D, seed=36)])
    # the queries sit S positions after kv_prev: own block causal window W, previous block the band (W - S, S)
    k_all, v_all = torch.cat([kv_prev[0], kv_own[0]], 1), torch.cat([kv_prev[1], kv_own[1]], 1)
    ro, rl, rdq, rdk, rdv = attn_fwd_bwd(q, k_all, v_all, do, SCALE, (W, 0), True)
    acc = torch.zeros(B, S, Hq, D, dtype=torch.float32, device=dev)
    lse = torch.full((B, Hq, S), float("-inf"), dtype=torch.float64, device=dev)
    qd, dod, prev_d, own_d = q.to(dev), do.to(dev), kv_prev.to(dev), kv_own.to(dev)
    flash_attn_fwd_func(qd, own_d, SCALE, (W, 0), True, acc, lse)
    flash_attn_fwd_func(qd, prev_d, SCALE, (W - S, S), False, acc, lse)
    assert_close("out", acc, ro)
    assert_lse_close(lse, rl)
    out, lse32 = acc.to(torch.bfloat16), lse.float()
    dq_a, dq_b = torch.empty_like(qd), torch.empty_like(qd)
    dkv_own, dkv_prev = torch.empty_like(own_d), torch.empty_like(prev_d)
    flash_attn_bwd_func(qd, own_d, out, lse32, dod, dq_a, dkv_own, SCALE, (W, 0), True)
    flash_attn_bwd_func(qd, prev_d, out, lse32, dod, dq_b, dkv_prev, SCALE, (W - S, S), False)
    assert_close("dq", dq_a.float() + dq_b.float(), rdq)
    assert_close("dk", torch.cat([dkv_prev[0], dkv_own[0]], 1), rdk)
    assert_close("dv", torch.cat([dkv_prev[1], dkv_own[1]], 1), rdv)


@pytest.mark.parametrize("window,causal", [((40, 88), False), ((40, 88), True), ((-1, -1), True), ((-1, 30), False)])
def test_flash_attn_funcs_more_queries_than_keys(window, causal):
    """q_len > kv_len and not plain full attention: leading queries see every key, trailing ones the
    window, both parts with causal=False whatever the caller passed (ring_swa/ops/attn.py:21, 38-60)."""
    from ring_swa.ops import flash_attn_bwd_func, flash_attn_fwd_func
    B, Sq, Sk, H = 1, 300, 128, 2
    dev = _dev()
    q, do = randn_bf16(B, Sq, H, D, seed=41), randn_bf16(B, Sq, H, D, seed=44)
    kv = torch.stack([randn_bf16(B, Sk, H, D, seed=42), randn_bf16(B, Sk, H, D, seed=43)])
    qf, kf, vf = (t.detach().float().requires_grad_(True) for t in (q, kv[0], kv[1]))
    o_head, l_head = attn(qf[:, :-Sk], kf, vf, SCALE, (-1, -1), False)
    o_tail, l_tail = attn(qf[:, -Sk:], kf, vf, SCALE, window, False)
    ro, rl = torch.cat([o_head, o_tail], 1), torch.cat([l_head, l_tail], 2)
    ro.backward(do.float())
    acc = torch.zeros(B, Sq, H, D, dtype=torch.float32, device=dev)
    lse = torch.full((B, H, Sq), float("-inf"), dtype=torch.float32, device=dev)
    qd, dod, kvd = q.to(dev), do.to(dev), kv.to(dev)
    flash_attn_fwd_func(qd, kvd, SCALE, window, causal, acc, lse)
    assert_close("out", acc, ro.detach())
    assert_lse_close(lse, rl.detach())
    dq, dkv = torch.empty_like(qd), torch.empty_like(kvd)
    flash_attn_bwd_func(qd, kvd, acc.to(torch.bfloat16), lse, dod, dq, dkv, SCALE, window, causal)
    assert_close("dq", dq, qf.grad)
    assert_close("dk", dkv[0], kf.grad)
    assert_close("dv", dkv[1], vf.grad)


def test_flash_attn_varlen_funcs_accumulate_and_differentiate():
    """flash_attn_varlen_fwd_func folds a packed partial result into the caller's accumulators (leading
    batch of 1, float32 output / float64 lse as the reference's ring keeps them), flash_attn_varlen_bwd_func
    writes dq and the stacked dkv (ring_swa/ops/attn.py:129-196): the diagonal call over shared boundaries
    and the rectangular off-diagonal call, merged, equal attention over both key blocks."""
    from ring_swa.ops import flash_attn_varlen_bwd_func, flash_attn_varlen_fwd_func
    Hq, Hkv, W = 4, 2, 48
    lens = [70, 1, 129]
    cu = [0]
    for L in lens:
        cu.append(cu[-1] + L)
    T = cu[-1]
    dev = _dev()
    q, do = randn_bf16(1, T, Hq, D, seed=51), randn_bf16(1, T, Hq, D, seed=54)
    kv = torch.stack([randn_bf16(1, T, Hkv, D, seed=52), randn_bf16(1, T, Hkv, D, seed=53)])
    window, causal = (W, 0), True
    ro, rl, rdq, rdk, rdv = _packed_reference(q[0], kv[0, 0], kv[1, 0], do[0], cu, cu, window, causal)
    cud = torch.tensor(cu, dtype=torch.int32, device=dev)
    acc = torch.zeros(1, T, Hq, D, dtype=torch.float32, device=dev)
    lse = torch.full((1, Hq, T), float("-inf"), dtype=torch.float64, device=dev)
    qd, dod, kvd = q.to(dev), do.to(dev), kv.to(dev)
    flash_attn_varlen_fwd_func(qd, kvd, SCALE, window, cud, cud, max(lens), max(lens), causal, acc, lse)
    assert_close("out", acc[0], ro)
    assert_lse_close(lse[0], rl)
    # a second call accumulates: the same keys again double every weight, out stays, lse grows by log 2
    flash_attn_varlen_fwd_func(qd, kvd, SCALE, window, cud, cud, max(lens), max(lens), causal, acc, lse)
    assert_close("out (merged twice)", acc[0], ro)
    assert_lse_close(lse[0], rl + 0.6931471805599453)
    dq, dkv = torch.empty_like(qd), torch.empty_like(kvd)
    flash_attn_varlen_bwd_func(qd, kvd, acc.to(torch.bfloat16), torch.as_tensor(rl, device=dev).float()[None], dod, dq, dkv,
                               cud, cud, max(lens), max(lens), SCALE, window, causal)
    assert_close("dq", dq[0], rdq)
    assert_close("dk", dkv[0, 0], rdk)
    assert_close("dv", dkv[1, 0], rdv)
    # different query / key boundaries (the off-diagonal hop of the packed ring): one launch per sequence
    cu_k = [0, 40, 41, 100]
    kv2 = torch.stack([randn_bf16(1, 100, Hkv, D, seed=55), randn_bf16(1, 100, Hkv, D, seed=56)])
    ro2, rl2, rdq2, rdk2, rdv2 = _packed_reference(q[0], kv2[0, 0], kv2[1, 0], do[0], cu, cu_k, (30, 10), False)
    ckd = torch.tensor(cu_k, dtype=torch.int32, device=dev)
    acc2 = torch.zeros_like(acc)
    lse2 = torch.full((1, Hq, T), float("-inf"), dtype=torch.float32, device=dev)
    flash_attn_varlen_fwd_func(qd, kv2.to(dev), SCALE, (30, 10), cud, ckd, max(lens), 59, False, acc2, lse2)
    assert_close("out (rect)", acc2[0], ro2)
    assert_lse_close(lse2[0], rl2)
    dq2, dkv2 = torch.empty_like(qd), torch.empty_like(kv2.to(dev))
    flash_attn_varlen_bwd_func(qd, kv2.to(dev), acc2.to(torch.bfloat16), lse2, dod, dq2, dkv2, cud, ckd, max(lens), 59,
                               SCALE, (30, 10), False)
    assert_close("dq (rect)", dq2[0], rdq2)
    assert_close("dk (rect)", dkv2[0, 0], rdk2)
    assert_close("dv (rect)", dkv2[1, 0], rdv2)
