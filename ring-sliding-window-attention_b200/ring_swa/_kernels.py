"""Torch-tensor front end of the C ABI: builds the parameter structs and launches on the current stream.

All tensors are 4-D here, [batch, tokens, heads, 128]; packed (varlen) callers add a leading batch of 1.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import torch

from . import _C

HEAD_DIM = 128
TILE = _C.TILE


@dataclass
class KVSpan:
    """A run of consecutive tokens' K/V held in one buffer (own tokens, a received halo, the sink)."""
    k: torch.Tensor                     # [B, L, Hkv, D]
    v: torch.Tensor
    pos_start: int                      # global position of token 0
    dk: Optional[torch.Tensor] = None   # backward outputs, same shape; fp32 or the input dtype
    dv: Optional[torch.Tensor] = None

    @property
    def length(self) -> int:
        return self.k.shape[1]


_status = {}

# Number of kernels of this library launched so far (benchmarks report the count per timed region).
launch_count = 0

# When set to a list, every rswa_bwd call records three fresh timing events, appended here as raw handles
# (start, mid, stop): start..mid brackets the dK/dV kernel, mid..stop the dQ kernel; benchmarks read them
# with rswa_event_elapsed_ms.
bwd_main_events = None
# Same for the forward kernel (one launch per rswa_fwd call).
fwd_events = None
_mid_event = {}   # per (device, stream): the event a one-call ring backward records between its two kernels


def _dev_key(device: torch.device):
    """('cuda', index) with a bare "cuda" resolved to the current device, so that every spelling of a
    device names the same status word."""
    index = device.index if device.index is not None else torch.cuda.current_device()
    return (device.type, index)


def status_word(device: torch.device) -> torch.Tensor:
    """Device word the kernels raise when a bounded device-side wait runs out."""
    key = _dev_key(device)
    device = torch.device(*key)
    if key not in _status:
        _status[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _status[key]


def check_device_status(device: Optional[torch.device] = None) -> None:
    """Synchronises and raises if any kernel reported a device-side time-out since the last check."""
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device())
    w = status_word(device)
    code = int(w.item())
    if code != 0:
        w.zero_()
        raise RuntimeError(f"ring_swa kernel reported device-side error code {code} (a bounded wait ran out)")


class _StatusMirror:
    """Pinned host copy of a device's status word, refreshed asynchronously after a backward."""

    def __init__(self, device: torch.device):
        self.host = torch.zeros(1, dtype=torch.int32).pin_memory()
        self.event = torch.cuda.Event()
        self.pending = False


_mirrors = {}


def _mirror(device: torch.device) -> _StatusMirror:
    key = _dev_key(device)
    if key not in _mirrors:
        _mirrors[key] = _StatusMirror(device)
    return _mirrors[key]


def mirror_status(device: torch.device) -> None:
    """Enqueues a copy of the status word to pinned host memory behind the kernels launched so far.

    The word is sticky on the device (kernels that start after it was raised do no work), so the
    host has to learn of it without a synchronisation in the hot loop: the public functions call
    this after every backward and raise_if_reported() at the start of the next call.  Skipped
    inside a stream capture."""
    if torch.cuda.is_current_stream_capturing():
        return
    m = _mirror(device)
    m.host.copy_(status_word(device), non_blocking=True)
    m.event.record()
    m.pending = True


def raise_if_reported(device: torch.device, wait: bool = False) -> None:
    """Raises RuntimeError if the last mirrored status word was non-zero, and clears the word so that
    the following call runs normally.  Without `wait` a copy still in flight is left for later."""
    m = _mirrors.get(_dev_key(device))
    if m is None or not m.pending or torch.cuda.is_current_stream_capturing():
        return
    if wait:
        m.event.synchronize()
    elif not m.event.query():
        return
    m.pending = False
    code = int(m.host[0])
    if code != 0:
        m.host.zero_()
        status_word(device).zero_()
        raise RuntimeError(f"ring_swa: a kernel of an earlier call gave up on a bounded device-side wait "
                           f"(code {code}); the results of that call are invalid. The status word has been "
                           f"cleared, later calls run normally.")


def _dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.bfloat16:
        return _C.DTYPE_BF16
    if t.dtype == torch.float16:
        return _C.DTYPE_FP16
    raise ValueError(f"ring_swa kernels take bfloat16 or float16 tensors, got {t.dtype}")


def _check4(name: str, t: torch.Tensor) -> None:
    if t.dim() != 4 or t.shape[-1] != HEAD_DIM:
        raise ValueError(f"{name} must be [batch, tokens, heads, {HEAD_DIM}], got {tuple(t.shape)}")
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor: ring_swa has no CPU path")
    if t.stride(-1) != 1:
        raise ValueError(f"{name} must be contiguous in the head dimension")


def _stream() -> C.c_void_p:
    # the raw handle of torch's current stream without building a Stream object: this runs a dozen times per
    # step and the Python-level getter costs ~15 us a call
    return C.c_void_p(torch._C._cuda_getCurrentRawStream(torch._C._cuda_getDevice()))


def _fill_geom(g: _C.Geom, q: torch.Tensor, spans: Sequence[KVSpan], window: int, n_sink: int, scale: float,
               q_pos_start: int, cu_seqlens: Optional[torch.Tensor], grads: bool) -> None:
    if len(spans) > _C.RSWA_MAX_SPANS:
        raise ValueError(f"at most {_C.RSWA_MAX_SPANS} KV spans per call")
    B, S, Hq, D = q.shape
    g.dtype = _dtype_code(q)
    g.batch, g.q_len, g.n_q_heads, g.head_dim = B, S, Hq, D
    g.n_kv_heads = spans[0].k.shape[2] if spans else Hq
    g.q_pos_start = int(q_pos_start)
    g.window = int(window)
    g.n_sink = int(n_sink)
    g.softmax_scale = float(scale)
    if cu_seqlens is not None:
        if cu_seqlens.dtype != torch.int32 or not cu_seqlens.is_cuda or not cu_seqlens.is_contiguous():
            raise ValueError("cu_seqlens must be a contiguous int32 CUDA tensor")
        g.cu_seqlens = cu_seqlens.data_ptr()
        g.n_seqs = cu_seqlens.numel() - 1
    else:
        g.cu_seqlens = None
        g.n_seqs = 0
    g.n_spans = len(spans)
    for i, s in enumerate(spans):
        _check4("k", s.k)
        _check4("v", s.v)
        if s.k.dtype != q.dtype or s.v.dtype != q.dtype:
            raise ValueError("q, k and v must have the same dtype")
        if s.k.shape != s.v.shape or s.k.stride() != s.v.stride():
            raise ValueError("k and v of a span must have the same shape and strides")
        if s.k.shape[0] != B or s.k.shape[2] != g.n_kv_heads:
            raise ValueError("span batch / head count mismatch")
        c = g.spans[i]
        c.k, c.v = s.k.data_ptr(), s.v.data_ptr()
        c.kv_stride_b, c.kv_stride_t, c.kv_stride_h = s.k.stride(0), s.k.stride(1), s.k.stride(2)
        c.pos_start, c.len = int(s.pos_start), s.k.shape[1]
        if grads and (s.dk is not None or s.dv is not None):
            if s.dk is None or s.dv is None:
                raise ValueError("dk and dv of a span must be given together")
            if s.dk.shape != s.k.shape or s.dv.shape != s.k.shape or s.dk.stride() != s.dv.stride():
                raise ValueError("dk/dv must match k in shape and each other in strides")
            if s.dk.dtype != s.dv.dtype or s.dk.dtype not in (torch.float32, q.dtype):
                raise ValueError("dk/dv must be float32 or the input dtype")
            c.dk, c.dv = s.dk.data_ptr(), s.dv.data_ptr()
            c.dkv_stride_b, c.dkv_stride_t, c.dkv_stride_h = s.dk.stride(0), s.dk.stride(1), s.dk.stride(2)
            c.grad_fp32 = 1 if s.dk.dtype == torch.float32 else 0


def fwd(q: torch.Tensor, spans: Sequence[KVSpan], window: int, n_sink: int, scale: float, q_pos_start: int = 0,
        cu_seqlens: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
        lse: Optional[torch.Tensor] = None, q_tiles: Optional[Tuple[int, int]] = None, carry: bool = False
        ) -> Tuple[torch.Tensor, torch.Tensor]:
    """out [B,S,Hq,D] (input dtype) and lse [B,Hq,S] (fp32) over the given spans.  With `carry`, out and
    lse (both required then) hold a partial result over other keys, which this call continues in place."""
    _check4("q", q)
    B, S, Hq, D = q.shape
    if carry and (out is None or lse is None):
        raise ValueError("carry needs the out and lse of the partial result to continue")
    if out is None:
        out = torch.empty((B, S, Hq, D), dtype=q.dtype, device=q.device)
    if lse is None:
        lse = torch.empty((B, Hq, S), dtype=torch.float32, device=q.device)
    p = _C.FwdParams()
    p.carry = 1 if carry else 0
    _fill_geom(p.g, q, spans, window, n_sink, scale, q_pos_start, cu_seqlens, grads=False)
    p.q = q.data_ptr()
    p.q_stride_b, p.q_stride_t, p.q_stride_h = q.stride(0), q.stride(1), q.stride(2)
    p.out = out.data_ptr()
    p.o_stride_b, p.o_stride_t, p.o_stride_h = out.stride(0), out.stride(1), out.stride(2)
    if lse.dtype != torch.float32 or lse.stride(2) != 1:
        raise ValueError("lse must be float32 [B, Hq, S] with contiguous tokens")
    p.lse = lse.data_ptr()
    p.lse_stride_b, p.lse_stride_h = lse.stride(0), lse.stride(1)
    p.q_tile_begin, p.q_tile_end = (0, 0) if q_tiles is None else (int(q_tiles[0]), int(q_tiles[1]))
    if q_tiles is not None and q_tiles[1] <= q_tiles[0]:
        return out, lse
    p.status = status_word(q.device).data_ptr()
    if fwd_events is not None:
        e0, e1 = _C.lib().rswa_event_create(), _C.lib().rswa_event_create()
        fwd_events.append((e0, e1))
        _C.lib().rswa_event_record(e0, _stream())
    _C.check(_C.lib().rswa_fwd(C.byref(p), _stream()), "rswa_fwd")
    if fwd_events is not None:
        _C.lib().rswa_event_record(e1, _stream())
    global launch_count
    launch_count += 1
    return out, lse


def bwd_workspace(q: torch.Tensor) -> torch.Tensor:
    B, S, Hq, D = q.shape
    n = _C.lib().rswa_bwd_workspace_bytes(B, S, Hq, D)
    if n < 0:
        raise ValueError("rswa_bwd_workspace_bytes: unsupported shape")
    return torch.empty(n, dtype=torch.uint8, device=q.device)


def bwd(q: torch.Tensor, spans: Sequence[KVSpan], out: torch.Tensor, lse: torch.Tensor, dout: torch.Tensor,
        dq: torch.Tensor, window: int, n_sink: int, scale: float, q_pos_start: int = 0,
        cu_seqlens: Optional[torch.Tensor] = None, workspace: Optional[torch.Tensor] = None,
        flags: int = _C.BWD_INIT | _C.BWD_FINISH, mid_event: Optional[int] = None) -> torch.Tensor:
    """K/V gradients of the spans that carry dk/dv buffers, and (with BWD_FINISH) dq summed over ALL given
    spans.  A ring rank calls it twice: the received spans first (INIT; their gradients leave early), then
    every span again with gradient buffers on the local one only (FINISH) -- or once with `mid_event`
    (from mid_event_for): the call records that event between the dK/dV kernel and the dQ kernel, so that
    another stream can pick the K/V gradients up while dQ is computed.  Returns the workspace."""
    for name, t in (("q", q), ("out", out), ("dout", dout), ("dq", dq)):
        _check4(name, t)
        if t.dtype != q.dtype or t.shape != q.shape:
            raise ValueError(f"{name} must match q in dtype and shape")
    if workspace is None:
        workspace = bwd_workspace(q)
    p = _C.BwdParams()
    _fill_geom(p.g, q, spans, window, n_sink, scale, q_pos_start, cu_seqlens, grads=True)
    p.q = q.data_ptr()
    p.q_stride_b, p.q_stride_t, p.q_stride_h = q.stride(0), q.stride(1), q.stride(2)
    p.out = out.data_ptr()
    p.o_stride_b, p.o_stride_t, p.o_stride_h = out.stride(0), out.stride(1), out.stride(2)
    p.dout = dout.data_ptr()
    p.do_stride_b, p.do_stride_t, p.do_stride_h = dout.stride(0), dout.stride(1), dout.stride(2)
    if lse.dtype != torch.float32 or lse.stride(2) != 1:
        raise ValueError("lse must be float32 [B, Hq, S] with contiguous tokens")
    p.lse = lse.data_ptr()
    p.lse_stride_b, p.lse_stride_h = lse.stride(0), lse.stride(1)
    p.dq = dq.data_ptr()
    p.dq_stride_b, p.dq_stride_t, p.dq_stride_h = dq.stride(0), dq.stride(1), dq.stride(2)
    p.workspace = workspace.data_ptr()
    p.workspace_bytes = workspace.numel()
    p.flags = int(flags)
    p.status = status_word(q.device).data_ptr()
    if mid_event is not None:
        p.ev_main_mid = mid_event
    if bwd_main_events is not None:
        p.ev_main_start, p.ev_main_stop = (_C.lib().rswa_event_create() for _ in range(2))
        if mid_event is None:
            p.ev_main_mid = _C.lib().rswa_event_create()
        bwd_main_events.append((p.ev_main_start, p.ev_main_mid, p.ev_main_stop))
    _C.check(_C.lib().rswa_bwd(C.byref(p), _stream()), "rswa_bwd")
    global launch_count
    launch_count += ((1 if flags & _C.BWD_INIT else 0) + (1 if any(s.dk is not None for s in spans) else 0) +
                     (1 if flags & _C.BWD_FINISH else 0))
    return workspace


def mid_event_for(device: torch.device) -> int:
    """The event (raw handle) to hand to bwd(mid_event=...) on this device's current stream: one per
    (device, stream), recorded anew by every call -- a stream that waits for it (stream_wait_event) right
    after the call sees that call's record or a later one of the same stream, behind which the call's
    dK/dV kernel has finished either way.  While benchmarks collect per-kernel times every call gets an
    event of its own, because they read the times later."""
    if bwd_main_events is not None:
        return _C.lib().rswa_event_create()
    key = _dev_key(device) + (_stream().value,)
    ev = _mid_event.get(key)
    if ev is None:
        with torch.cuda.device(device):
            ev = _C.lib().rswa_event_create()
        if not ev:
            raise RuntimeError("rswa_event_create failed")
        _mid_event[key] = ev
    return ev


def stream_wait_event(stream: torch.cuda.Stream, event: int) -> None:
    _C.check(_C.lib().rswa_event_wait(C.c_void_p(event), C.c_void_p(stream.cuda_stream)), "rswa_event_wait")


def bwd_noalloc(q: torch.Tensor, spans: Sequence[KVSpan], out: torch.Tensor, lse: torch.Tensor,
                dout: torch.Tensor, dq: torch.Tensor, window: int, n_sink: int, scale: float,
                q_pos_start: int = 0, cu_seqlens: Optional[torch.Tensor] = None) -> None:
    """A whole backward through rswa_bwd_noalloc: no workspace tensor is created or passed.

    For integrations that may not allocate device memory where they call the backward (they only
    hold the operator's own tensors, or allocation is forbidden after start-up): the scratch is
    the fixed array (64 MiB + 256 bytes) inside librswa.so.  Raises ValueError when the problem is too large
    for it.  Calls on one device share that array, so they must not overlap on the GPU.
    """
    for name, t in (("q", q), ("out", out), ("dout", dout), ("dq", dq)):
        _check4(name, t)
        if t.dtype != q.dtype or t.shape != q.shape:
            raise ValueError(f"{name} must match q in dtype and shape")
    if lse.dtype != torch.float32 or lse.stride(2) != 1:
        raise ValueError("lse must be float32 [B, Hq, S] with contiguous tokens")
    p = _C.BwdParams()
    _fill_geom(p.g, q, spans, window, n_sink, scale, q_pos_start, cu_seqlens, grads=True)
    p.q = q.data_ptr()
    p.q_stride_b, p.q_stride_t, p.q_stride_h = q.stride(0), q.stride(1), q.stride(2)
    p.out = out.data_ptr()
    p.o_stride_b, p.o_stride_t, p.o_stride_h = out.stride(0), out.stride(1), out.stride(2)
    p.dout = dout.data_ptr()
    p.do_stride_b, p.do_stride_t, p.do_stride_h = dout.stride(0), dout.stride(1), dout.stride(2)
    p.lse = lse.data_ptr()
    p.lse_stride_b, p.lse_stride_h = lse.stride(0), lse.stride(1)
    p.dq = dq.data_ptr()
    p.dq_stride_b, p.dq_stride_t, p.dq_stride_h = dq.stride(0), dq.stride(1), dq.stride(2)
    p.status = status_word(q.device).data_ptr()
    _C.check(_C.lib().rswa_bwd_noalloc(C.byref(p), _stream()), "rswa_bwd_noalloc")
    global launch_count
    launch_count += 2 + (1 if spans else 0)


def merge(o_a: torch.Tensor, lse_a: torch.Tensor, o_b: torch.Tensor, lse_b: torch.Tensor,
          out: Optional[torch.Tensor] = None, lse_out: Optional[torch.Tensor] = None
          ) -> Tuple[torch.Tensor, torch.Tensor]:
    """Log-sum-exp merge of two partial results; in place on (o_a, lse_a) unless outputs are given."""
    _check4("o_a", o_a)
    _check4("o_b", o_b)
    out = o_a if out is None else out
    lse_out = lse_a if lse_out is None else lse_out
    B, S, H, D = o_a.shape
    for l in (lse_a, lse_b, lse_out):
        if l.dtype != torch.float32 or l.shape != (B, H, S) or l.stride() != lse_a.stride() or l.stride(2) != 1:
            raise ValueError("lse tensors must be float32 [B, H, S] with identical strides")
    p = _C.MergeParams()
    p.dtype = _dtype_code(o_a)
    p.batch, p.q_len, p.n_heads, p.head_dim = B, S, H, D
    p.o_a, p.o_b, p.o = o_a.data_ptr(), o_b.data_ptr(), out.data_ptr()
    p.oa_stride_b, p.oa_stride_t, p.oa_stride_h = o_a.stride(0), o_a.stride(1), o_a.stride(2)
    p.ob_stride_b, p.ob_stride_t, p.ob_stride_h = o_b.stride(0), o_b.stride(1), o_b.stride(2)
    p.o_stride_b, p.o_stride_t, p.o_stride_h = out.stride(0), out.stride(1), out.stride(2)
    p.lse_a, p.lse_b, p.lse = lse_a.data_ptr(), lse_b.data_ptr(), lse_out.data_ptr()
    p.lse_stride_b, p.lse_stride_h = lse_a.stride(0), lse_a.stride(1)
    _C.check(_C.lib().rswa_merge(C.byref(p), _stream()), "rswa_merge")
    global launch_count
    launch_count += 1
    return out, lse_out


def merge_acc(acc_o: torch.Tensor, acc_lse: torch.Tensor, new_o: torch.Tensor, new_lse: torch.Tensor) -> None:
    """In-place merge of a partial result into a float32 accumulator with a float32 or float64 lse."""
    if acc_o.dim() != 4 or new_o.shape != acc_o.shape:
        raise ValueError("merge_acc: outputs must be [B, S, H, D] of one shape")
    if acc_o.dtype != torch.float32 or acc_o.stride(3) != 1 or new_o.stride(3) != 1:
        raise ValueError("merge_acc: the accumulator must be float32; head_dim must be contiguous in both")
    if acc_lse.dtype not in (torch.float32, torch.float64) or new_lse.dtype != torch.float32:
        raise ValueError("merge_acc: acc lse must be float32/float64 and the incoming lse float32")
    B, S, H, D = acc_o.shape
    for l in (acc_lse, new_lse):
        if l.shape != (B, H, S) or l.stride(2) != 1:
            raise ValueError("merge_acc: lse tensors must be [B, H, S] with contiguous tokens")
    p = _C.MergeAccParams()
    p.new_dtype = _C.DTYPE_F32 if new_o.dtype == torch.float32 else _dtype_code(new_o)
    p.lse_f64 = 1 if acc_lse.dtype == torch.float64 else 0
    p.batch, p.q_len, p.n_heads, p.head_dim = B, S, H, D
    p.acc_o, p.new_o = acc_o.data_ptr(), new_o.data_ptr()
    p.acc_stride_b, p.acc_stride_t, p.acc_stride_h = acc_o.stride(0), acc_o.stride(1), acc_o.stride(2)
    p.new_stride_b, p.new_stride_t, p.new_stride_h = new_o.stride(0), new_o.stride(1), new_o.stride(2)
    p.acc_lse, p.new_lse = acc_lse.data_ptr(), new_lse.data_ptr()
    p.acc_lse_stride_b, p.acc_lse_stride_h = acc_lse.stride(0), acc_lse.stride(1)
    p.new_lse_stride_b, p.new_lse_stride_h = new_lse.stride(0), new_lse.stride(1)
    _C.check(_C.lib().rswa_merge_acc(C.byref(p), _stream()), "rswa_merge_acc")
    global launch_count
    launch_count += 1


def _rows(t: torch.Tensor) -> Tuple[int, int, int]:
    """(batch, batch stride, contiguous elements per batch row) of a [B, ...] tensor."""
    if t.dim() < 2 or not t[0].is_contiguous():
        raise ValueError("expected a tensor whose batch rows are contiguous")
    return t.shape[0], t.stride(0), t[0].numel()


def halo_accumulate(acc: torch.Tensor, recv: torch.Tensor) -> None:
    """acc (fp32) += recv, both [B, L, H, D] with contiguous batch rows."""
    if acc.dtype != torch.float32 or acc.shape != recv.shape:
        raise ValueError("halo_accumulate: acc must be float32 and match recv in shape")
    B, asb, n = _rows(acc)
    _, rsb, _ = _rows(recv)
    code = _C.DTYPE_F32 if recv.dtype == torch.float32 else _dtype_code(recv)
    _C.check(_C.lib().rswa_halo_accumulate(acc.data_ptr(), asb, recv.data_ptr(), rsb, code, B, n, _stream()),
             "rswa_halo_accumulate")
    global launch_count
    launch_count += 1


def halo_accumulate_cast(dst: torch.Tensor, acc: torch.Tensor, recv: torch.Tensor) -> None:
    """dst (16-bit) = round(acc + recv); acc (fp32) is not written.  All [B, ...] with contiguous batch rows."""
    if acc.dtype != torch.float32 or acc.shape != recv.shape or dst.shape != acc.shape:
        raise ValueError("halo_accumulate_cast: acc must be float32 and match recv and dst in shape")
    B, asb, n = _rows(acc)
    _, rsb, _ = _rows(recv)
    _, dsb, _ = _rows(dst)
    code = _C.DTYPE_F32 if recv.dtype == torch.float32 else _dtype_code(recv)
    _C.check(_C.lib().rswa_halo_accumulate_cast(dst.data_ptr(), dsb, _dtype_code(dst), acc.data_ptr(), asb, recv.data_ptr(),
                                                rsb, code, B, n, _stream()), "rswa_halo_accumulate_cast")
    global launch_count
    launch_count += 1


def cast_from_f32(dst: torch.Tensor, src: torch.Tensor) -> None:
    if src.dtype != torch.float32 or dst.shape != src.shape:
        raise ValueError("cast_from_f32: src must be float32 and match dst in shape")
    B, dsb, n = _rows(dst)
    _, ssb, _ = _rows(src)
    _C.check(_C.lib().rswa_cast_from_f32(dst.data_ptr(), dsb, src.data_ptr(), ssb, _dtype_code(dst), B, n,
                                         _stream()), "rswa_cast_from_f32")
    global launch_count
    launch_count += 1


def peer_put(dst_ptr: int, dst_pitch: int, src: torch.Tensor, flag_ptr: int, value: int) -> None:
    """Copy-engine transfer of src ([rows, ...] with contiguous rows, local) to dst_ptr (local or a mapped
    peer address, rows dst_pitch bytes apart) on the current stream, then release `value` into the flag
    word at flag_ptr (0: no flag)."""
    rows, sb, n = _rows(src)
    es = src.element_size()
    _C.check(_C.lib().rswa_peer_put(dst_ptr, int(dst_pitch), src.data_ptr(), sb * es if rows > 1 else n * es, n * es, rows,
                                    flag_ptr if flag_ptr else None, int(value), _stream()), "rswa_peer_put")
    global launch_count
    launch_count += 1 if flag_ptr else 0


def flag_set(flag_ptr: int, value: int) -> None:
    _C.check(_C.lib().rswa_flag_set(flag_ptr, int(value), _stream()), "rswa_flag_set")
    global launch_count
    launch_count += 1


def flag_wait(flag_ptr: int, value: int, device: torch.device, timeout_s: float = 5.0) -> None:
    """Everything launched on the current stream after this starts once the flag has reached `value`; if it
    has not within timeout_s, the device status word is raised instead (see check_device_status)."""
    _C.check(_C.lib().rswa_flag_wait(flag_ptr, int(value), status_word(device).data_ptr(), int(timeout_s * 1e9),
                                     _stream()), "rswa_flag_wait")
    global launch_count
    launch_count += 1


def selftest_mma(mode: int, a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    d = torch.zeros(128, 128, dtype=torch.float32, device=a.device)
    _C.check(_C.lib().rswa_selftest_mma(mode, a.data_ptr(), b.data_ptr(), d.data_ptr(),
                                        status_word(a.device).data_ptr(), _stream()), "rswa_selftest_mma")
    return d
