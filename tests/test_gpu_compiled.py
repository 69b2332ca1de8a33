"""The registered custom operators (ring_swa.compiled): operator checks, tracing with torch.compile,
and a forward + backward replayed from a CUDA graph, all against the eager public API."""
import pytest
import torch

from gpu_util import assert_close, randn_bf16

pytestmark = pytest.mark.gpu

D = 128


def _inputs(B=1, S=384, Hq=4, Hkv=2, seed=0):
    dev = torch.device("cuda")
    q, do = randn_bf16(B, S, Hq, D, seed=seed).to(dev), randn_bf16(B, S, Hq, D, seed=seed + 3).to(dev)
    k, v = randn_bf16(B, S, Hkv, D, seed=seed + 1).to(dev), randn_bf16(B, S, Hkv, D, seed=seed + 2).to(dev)
    return q, k, v, do


def _eager(q, k, v, do, W, n_sink=0):
    import ring_swa
    qq, kk, vv = (t.detach().clone().requires_grad_(True) for t in (q, k, v))
    if n_sink:
        out = ring_swa.ring_streaming_llm_attn(qq, kk, vv, W, num_sink_tokens=n_sink)
    else:
        out = ring_swa.ring_sliding_window_attn(qq, kk, vv, W)
    out.backward(do)
    return out.detach(), qq.grad, kk.grad, vv.grad


def test_operator_registration_checks():
    from ring_swa import compiled
    q, k, v, do = _inputs()
    torch.library.opcheck(compiled.swa_fwd, (q, k, v, 100, 0, D ** -0.5, None),
                          test_utils=("test_schema", "test_faketensor"))
    out, lse = compiled.swa_fwd(q, k, v, 100, 0, D ** -0.5, None)
    torch.library.opcheck(compiled.swa_bwd, (q, k, v, out, lse, do, 100, 0, D ** -0.5, None),
                          test_utils=("test_schema", "test_faketensor"))


@pytest.mark.parametrize("n_sink", [0, 1])
def test_matches_eager_api_and_traces(n_sink):
    from ring_swa import compiled
    W = 100
    q, k, v, do = _inputs(seed=10)
    ref = _eager(q, k, v, do, W, n_sink)

    def fn(a, b, c):
        return compiled.sliding_window_attn(a * 1.0, b, c, W, num_sink_tokens=n_sink)

    traced = torch.compile(fn, backend="aot_eager", fullgraph=True)   # one opaque node, no graph break
    for f in (fn, traced):
        qq, kk, vv = (t.detach().clone().requires_grad_(True) for t in (q, k, v))
        out = f(qq, kk, vv)
        out.backward(do)
        for name, got, want in zip(("out", "dq", "dk", "dv"), (out, qq.grad, kk.grad, vv.grad), ref):
            assert torch.equal(got.detach(), want), name       # same kernels, same bits


def test_packed_sequences():
    import ring_swa
    from ring_swa import compiled
    dev = torch.device("cuda")
    lens = [100, 37, 250]
    cu = torch.tensor([0, 100, 137, 387], dtype=torch.int32, device=dev)
    q, k, v, do = (t[0, :387] for t in _inputs(S=512, seed=20))
    qq, kk, vv = (t.detach().clone().requires_grad_(True) for t in (q, k, v))
    want = ring_swa.ring_sliding_window_attn_varlen(qq, kk, vv, 64, cu, cp_size=1)
    want.backward(do)
    q2, k2, v2 = (t.detach().clone().requires_grad_(True) for t in (q, k, v))
    got = compiled.sliding_window_attn(q2, k2, v2, 64, cu_seqlens=cu)
    got.backward(do)
    assert torch.equal(got, want) and torch.equal(q2.grad, qq.grad) and torch.equal(k2.grad, kk.grad)
    assert torch.equal(v2.grad, vv.grad)


def test_forward_and_backward_replay_from_a_cuda_graph():
    from ring_swa import compiled, _kernels
    W = 100
    q, k, v, do = _inputs(seed=30)
    ref = _eager(q, k, v, do, W)
    sq, sk, sv, sdo = (torch.zeros_like(t) for t in (q, k, v, do))
    # warm up on a side stream (first calls create the status word and bind the context)
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        for _ in range(2):
            o, l = compiled.swa_fwd(sq, sk, sv, W, 0, D ** -0.5, None)
            compiled.swa_bwd(sq, sk, sv, o, l, sdo, W, 0, D ** -0.5, None)
    torch.cuda.current_stream().wait_stream(s)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        o, l = compiled.swa_fwd(sq, sk, sv, W, 0, D ** -0.5, None)
        dq, dk, dv = compiled.swa_bwd(sq, sk, sv, o, l, sdo, W, 0, D ** -0.5, None)
    for t, src in zip((sq, sk, sv, sdo), (q, k, v, do)):
        t.copy_(src)
    graph.replay()
    torch.cuda.synchronize()
    _kernels.check_device_status()
    for name, got, want in zip(("out", "dq", "dk", "dv"), (o, dq, dk, dv), ref):
        assert torch.equal(got, want), name
    assert_close("out", o, ref[0])
