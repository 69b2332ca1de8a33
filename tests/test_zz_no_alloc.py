"""rswa_bwd_noalloc, the backward for hosts that cannot allocate device memory at the call site (they
are given the operator's tensors and nothing else, or allocation is off limits once the process has
started serving).  Called through the C ABI and compared with rswa_bwd on the same inputs, twice in a
row: the second call works in the same built-in scratch array and must not see the first call's sums.

This file sorts last on purpose, so that a run stopping at the first failure has run everything else.
"""
import pytest
import torch

from gpu_util import assert_close, randn_bf16

pytestmark = pytest.mark.gpu
D = 128


def _problem(seed, S, Hq, Hkv, W, n_sink, cu):
    from ring_swa import _kernels as K
    dev = torch.device("cuda")
    q = randn_bf16(1, S, Hq, D, seed=seed).to(dev)
    k = randn_bf16(1, S, Hkv, D, seed=seed + 1).to(dev)
    v = randn_bf16(1, S, Hkv, D, seed=seed + 2).to(dev)
    do = randn_bf16(1, S, Hq, D, seed=seed + 3).to(dev)
    cud = torch.tensor(cu, dtype=torch.int32, device=dev) if cu else None
    out, lse = K.fwd(q, [K.KVSpan(k, v, 0)], W, n_sink, D ** -0.5, 0, cud)
    return q, k, v, do, out, lse, cud


def _both(seed, S, Hq, Hkv, W, n_sink, cu):
    from ring_swa import _kernels as K
    q, k, v, do, out, lse, cud = _problem(seed, S, Hq, Hkv, W, n_sink, cu)
    ref = [torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)]
    K.bwd(q, [K.KVSpan(k, v, 0, dk=ref[1], dv=ref[2])], out, lse, do, ref[0], W, n_sink, D ** -0.5, 0, cud)
    got = [torch.full_like(q, float("nan")), torch.full_like(k, float("nan")), torch.full_like(v, float("nan"))]
    before = torch.cuda.memory_allocated()
    K.bwd_noalloc(q, [K.KVSpan(k, v, 0, dk=got[1], dv=got[2])], out, lse, do, got[0], W, n_sink, D ** -0.5, 0, cud)
    assert torch.cuda.memory_allocated() == before      # nothing came from torch's allocator either
    K.check_device_status()
    for name, a, b in zip(("dq", "dk", "dv"), got, ref):
        assert_close(name, a, b.float())
    # ... and, directly, against the CPU oracle
    from oracle.dense_attn import dense_attn_fwd_bwd
    _o, _l, odq, odk, odv = dense_attn_fwd_bwd(q.cpu(), k.cpu(), v.cpu(), do.cpu(), W, D ** -0.5, n_sink, cu)
    for name, a, b in zip(("dq", "dk", "dv"), got, (odq, odk, odv)):
        assert_close(name + " vs oracle", a, b)


def test_noalloc_backward_matches_twice_in_a_row():
    # first call: large values left behind in the shared scratch ...
    _both(seed=100, S=900, Hq=8, Hkv=2, W=200, n_sink=1, cu=None)
    # ... second call: another shape, packed sequences; must start from a clean accumulator
    _both(seed=200, S=515, Hq=4, Hkv=4, W=64, n_sink=0, cu=[0, 100, 101, 515])
    # and the same problem again
    _both(seed=200, S=515, Hq=4, Hkv=4, W=64, n_sink=0, cu=[0, 100, 101, 515])


def test_noalloc_rejects_what_does_not_fit():
    import ctypes
    from ring_swa import _C
    lib = _C.lib()
    assert lib.rswa_noalloc_scratch_bytes() == (64 << 20) + 256
    # geometry whose two fp32 rows per (batch, head, token) exceed the built-in array: rejected on the
    # host before anything is touched or launched, so small stand-in buffers are enough here
    dev = torch.device("cuda")
    buf = torch.zeros(1024, dtype=torch.bfloat16, device=dev)
    p = _C.BwdParams()
    p.g.dtype, p.g.head_dim = 0, D
    p.g.batch, p.g.q_len, p.g.n_q_heads, p.g.n_kv_heads = 8, 65536, 32, 32     # 16.8 M rows -> 128 MiB
    p.g.window, p.g.softmax_scale = 10, 0.1
    for name in ("q", "out", "dout", "lse", "dq", "status"):
        setattr(p, name, buf.data_ptr())
    rc = lib.rswa_bwd_noalloc(ctypes.byref(p), None)
    assert rc == -4 and b"scratch" in lib.rswa_last_error()
    with pytest.raises(ValueError, match="scratch"):
        _C.check(rc, "rswa_bwd_noalloc")


def test_noalloc_accepts_the_largest_documented_shape():
    """262144 tokens of 32 heads need exactly the array: the size check lets the call through.  The head
    counts do not divide, so the argument check that comes next rejects it before anything is launched
    (host-side only: the buffers are stand-ins)."""
    import ctypes
    from ring_swa import _C
    lib = _C.lib()
    assert lib.rswa_bwd_workspace_bytes(1, 262144, 32, D) == lib.rswa_noalloc_scratch_bytes()
    buf = torch.zeros(1024, dtype=torch.bfloat16, device="cuda")
    p = _C.BwdParams()
    p.g.dtype, p.g.head_dim = 0, D
    p.g.batch, p.g.q_len, p.g.n_q_heads, p.g.n_kv_heads = 1, 262144, 32, 5
    p.g.window, p.g.softmax_scale = 10, 0.1
    for name in ("q", "out", "dout", "lse", "dq", "status"):
        setattr(p, name, buf.data_ptr())
    rc = lib.rswa_bwd_noalloc(ctypes.byref(p), None)
    assert rc == -1 and b"divisible" in lib.rswa_last_error()
    p.g.q_len = 262144 + 1            # one more token: one more tile of rows, too large
    assert lib.rswa_bwd_noalloc(ctypes.byref(p), None) == -4
