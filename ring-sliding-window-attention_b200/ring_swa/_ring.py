"""The one autograd function behind the four public entry points.

Forward, on rank r of cp (sequence split contiguously, chunk i on group rank i):
  1. post the sink exchange and the halo exchange (torch.distributed P2P, NCCL over NVLink);
  2. while they fly, run the query tiles that only see local keys;
  3. when the halo has landed, run the remaining tiles over sink | halo | local in ONE pass
     (no per-hop partial results), or, when the window spans the whole chunk (W >= S), run the
     local keys first and let the halo pass continue that partial result inside the kernel.
Backward mirrors it: K/V gradients of halo (and remote sink) tokens are computed first and sent
back to their owners while the local part runs; the owner adds them in fp32 and rounds once.

This replaces RingSlidingWindowAttn / RingSlidingWindowAttnVarlen / RingStreamingLLMAttn /
RingStreamingLLMVarlen of the reference (ring_swa/sliding_window/nonvarlen.py:17-338,
varlen.py:19-359, ring_swa/streaming_llm/nonvarlen.py:20-397, varlen.py:20-473) and the naive
single-GPU StreamingLLM functions (ring_swa/streaming_llm/naive.py:11-210).
"""
from __future__ import annotations

import os
import sys
from dataclasses import dataclass
from typing import List, Optional, Sequence

import torch
import torch.distributed as dist

from . import _C
from . import _kernels as K
from . import _peer
from ._plan import RingPlan, make_plan

# Optional tracing: RING_SWA_NVTX=1 wraps the phases of a call in NVTX ranges (visible in a profiler's
# timeline), RING_SWA_DEBUG=1 logs each call's exchange plan on the host.  Both are off by default and
# cost one attribute test per phase then.
_NVTX = os.environ.get("RING_SWA_NVTX", "0") not in ("", "0")
_DEBUG = os.environ.get("RING_SWA_DEBUG", "0") not in ("", "0")


PHASES = ("fwd.local", "fwd.tiles_without_halo", "fwd.halo_wait", "fwd.tiles_with_halo", "fwd.halo_carried",
          "bwd.halo_spans", "bwd.local_and_dq", "bwd.grad_wait", "bwd.accumulate")
_phase_events = None   # list of (name, start event, stop event) while phase timing is on


def phase_timing(on: bool) -> None:
    """Starts (and clears) or stops the recording of one CUDA event pair around every phase on the
    compute stream.  Off by default; a measurement aid, the product path records nothing."""
    global _phase_events
    _phase_events = [] if on else None


def phase_times() -> dict:
    """{phase: total milliseconds on the compute stream} over the calls recorded since phase_timing(True)
    (synchronises).  `halo_wait` / `grad_wait` are the time the compute stream stood still for data."""
    out = {name: 0.0 for name in PHASES}
    if _phase_events:
        torch.cuda.synchronize()
        for name, e0, e1 in _phase_events:
            out[name] += e0.elapsed_time(e1)
    return out


class _phase:
    """with _phase("name"): an NVTX range when tracing is on, an event pair when phase timing is on,
    nothing otherwise."""

    def __init__(self, name: str):
        self.name = name

    def __enter__(self):
        if _NVTX:
            torch.cuda.nvtx.range_push("ring_swa." + self.name)
        if _phase_events is not None:
            self.e0 = torch.cuda.Event(enable_timing=True)
            self.e0.record()

    def __exit__(self, *exc):
        if _NVTX:
            torch.cuda.nvtx.range_pop()
        if _phase_events is not None:
            e1 = torch.cuda.Event(enable_timing=True)
            e1.record()
            _phase_events.append((self.name, self.e0, e1))
        return False


def _log_plan(what: str, plan, link) -> None:
    if _DEBUG:
        print(f"[ring_swa] {what}: rank {plan.rank}/{plan.cp} S={plan.seq_per_rank} W={plan.window} n_sink={plan.n_sink} "
              f"halo_recv={[(h.src, h.length) for h in plan.halo_recv]} halo_send={[(h.dst, h.length) for h in plan.halo_send]} "
              f"sink_recv={[(x.owner, x.n) for x in plan.sink_recv]} sink_send={[(x.dst, x.n) for x in plan.sink_send]} "
              f"halo_tiles=[0,{plan.halo_tile_end}) of {plan.n_tiles} halos_by={'peer stores' if link is not None else 'messages'}",
              file=sys.stderr, flush=True)


# dtype the halo / sink gradients travel in (None: the input dtype, like the per-hop partials of
# ring_swa/sliding_window/nonvarlen.py:194-195; torch.float32 to send them unrounded)
HALO_GRAD_WIRE_DTYPE = None


@dataclass
class RingCtx:
    """Who is where.  `group` is None on a single GPU."""
    group: Optional[dist.ProcessGroup]
    cp: int
    rank: int
    prev_global: Optional[int]
    next_global: Optional[int]
    chunk_lens: Optional[tuple] = None   # tokens per group rank where the chunks differ in length

    def global_rank(self, group_rank: int) -> int:
        if group_rank == self.rank + 1 and self.next_global is not None:
            return self.next_global
        if group_rank == self.rank - 1 and self.prev_global is not None:
            return self.prev_global
        return dist.get_global_rank(self.group, group_rank)


def _exchange(ops: List[dist.P2POp]) -> list:
    return list(dist.batch_isend_irecv(ops)) if ops else []


def _wait(works) -> None:
    """Waits for every request once and empties the list (a second wait on a finished gloo
    send/recv request blocks for ever, so the call must be idempotent)."""
    while works:
        works.pop().wait()


def _dense(t: torch.Tensor) -> torch.Tensor:
    """The kernels address tensors through TMA descriptors: strides must be positive multiples of
    16 bytes with the head dimension contiguous.  Anything else (expanded grads, odd slices) is copied."""
    ok = t.stride(-1) == 1 and all(st > 0 and st % 8 == 0 for st in t.stride()[:-1]) and t.data_ptr() % 16 == 0
    return t if ok else t.contiguous()


def _pack_tail(k4: torch.Tensor, v4: torch.Tensor, length: int) -> torch.Tensor:
    """[2, B, L, Hkv, D] copy of the trailing `length` tokens of K and V (one message, one copy kernel)."""
    S = k4.shape[1]
    return torch.stack((k4[:, S - length:], v4[:, S - length:]))


class RingAttn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, window: int, n_sink: int, softmax_scale: float,
                cu_seqlens: Optional[torch.Tensor], cu_host: Optional[Sequence[int]], ring: RingCtx):
        varlen = cu_seqlens is not None
        if q.is_cuda:
            K.raise_if_reported(q.device)  # a time-out reported by an earlier call's kernels
        q4, k4, v4 = (_dense(x).unsqueeze(0) if varlen else _dense(x) for x in (q, k, v))
        if v4.stride() != k4.stride():
            v4 = v4.contiguous()
            k4 = k4.contiguous()
        B, S, Hq, D = q4.shape
        plan = make_plan(ring.cp, ring.rank, S, window, n_sink, cu_host, ring.chunk_lens)
        if 1 + len(plan.halo_recv) + len(plan.sink_recv) > _C.RSWA_MAX_SPANS:
            raise ValueError("window reaches over more ranks than one call supports "
                             f"({len(plan.halo_recv)} hops)")
        pos0 = plan.q_pos_start
        local = K.KVSpan(k4, v4, pos0)

        # -- post the exchanges
        sink_ops, halo_ops, keep = [], [], []
        sink_spans = []
        for s in plan.sink_send:
            buf = torch.stack([k4[:, s.offset:s.offset + s.n], v4[:, s.offset:s.offset + s.n]])
            keep.append(buf)
            sink_ops.append(dist.P2POp(dist.isend, buf, ring.global_rank(s.dst), ring.group))
        for sr in plan.sink_recv:
            sbuf = torch.empty((2, B, sr.n) + tuple(k4.shape[2:]), dtype=k4.dtype, device=k4.device)
            sink_ops.append(dist.P2POp(dist.irecv, sbuf, ring.global_rank(sr.owner), ring.group))
            sink_spans.append(K.KVSpan(sbuf[0], sbuf[1], sr.pos_start))
        # Halo K/V: peer stores into the receivers' buffers where the ranks are GPUs of one node (no
        # communication kernel runs next to the attention kernels), torch.distributed messages otherwise.
        link = None
        if ring.cp > 1 and q4.is_cuda and _peer.wanted():
            lens = ring.chunk_lens or (S,)
            link = _peer.link_for(ring.group, q4.device, ring.cp, max(lens), window, B, k4.shape[2], D, min(lens))
        halo_spans = []
        halo_shape = lambda r: (2, B, r.length) + tuple(k4.shape[2:])  # noqa: E731
        if link is not None:
            ready = torch.cuda.Event()
            ready.record()
            for s in plan.halo_send:
                link.put(0, s.hop, s.dst, [k4[:, S - s.length:], v4[:, S - s.length:]], ready)
        else:
            packed = {}
            for s in plan.halo_send:
                if s.length not in packed:
                    packed[s.length] = _pack_tail(k4, v4, s.length)
                halo_ops.append(dist.P2POp(dist.isend, packed[s.length], ring.global_rank(s.dst), ring.group))
            for r in plan.halo_recv:
                hbuf = torch.empty(halo_shape(r), dtype=k4.dtype, device=k4.device)
                halo_ops.append(dist.P2POp(dist.irecv, hbuf, ring.global_rank(r.src), ring.group))
                halo_spans.append(K.KVSpan(hbuf[0], hbuf[1], r.pos_start))

        def halos_landed():
            """Behind this call on the current stream the halo spans hold their data."""
            _wait(halo_works)
            if link is not None and not halo_spans:
                for r in plan.halo_recv:
                    n = link.arrived(0, r.hop)
                    # out of the shared slot into a tensor of this call (the backward needs it again, and
                    # the sender may reuse the slot for its next message once it is told so)
                    hbuf = torch.empty(halo_shape(r), dtype=k4.dtype, device=k4.device)
                    hbuf.copy_(link.slot_view(0, r.hop, halo_shape(r), k4.dtype))
                    link.release(0, r.hop, r.src, n)
                    halo_spans.append(K.KVSpan(hbuf[0], hbuf[1], r.pos_start))

        sink_works = _exchange(sink_ops)
        halo_works = _exchange(halo_ops)

        # -- compute
        out = torch.empty_like(q4)
        lse = torch.empty((B, Hq, S), dtype=torch.float32, device=q4.device)
        args = dict(window=window, n_sink=n_sink, scale=softmax_scale, q_pos_start=pos0, cu_seqlens=cu_seqlens)
        _wait(sink_works)
        _log_plan("forward", plan, link)
        near = sink_spans + [local]
        if not plan.halo_recv:
            with _phase("fwd.local"):
                K.fwd(q4, near, out=out, lse=lse, **args)
        elif window < S:
            nb = plan.halo_tile_end
            with _phase("fwd.tiles_without_halo"):
                K.fwd(q4, near, out=out, lse=lse, q_tiles=(nb, plan.n_tiles), **args)
            with _phase("fwd.halo_wait"):
                halos_landed()
            spans = sink_spans + halo_spans[::-1] + [local]
            with _phase("fwd.tiles_with_halo"):
                K.fwd(q4, spans, out=out, lse=lse, q_tiles=(0, nb), **args)
        else:
            with _phase("fwd.local"):
                K.fwd(q4, near, out=out, lse=lse, **args)
            with _phase("fwd.halo_wait"):
                halos_landed()
            # the halo pass continues the local partial result inside the kernel (no second buffer, no
            # separate merge pass)
            with _phase("fwd.halo_carried"):
                K.fwd(q4, halo_spans[::-1], out=out, lse=lse, carry=True, **args)
        _wait(halo_works)

        ctx.save_for_backward(q4, k4, v4, out, lse, cu_seqlens,
                              *[t for s in halo_spans for t in (s.k, s.v)],
                              *[t for s in sink_spans for t in (s.k, s.v)])
        ctx.plan, ctx.ring, ctx.args, ctx.varlen, ctx.link = plan, ring, args, varlen, link
        return out.squeeze(0) if varlen else out

    @staticmethod
    def backward(ctx, dout):
        plan: RingPlan = ctx.plan
        ring: RingCtx = ctx.ring
        saved = ctx.saved_tensors
        q, k, v, out, lse, cu_seqlens = saved[:6]
        rest = list(saved[6:])
        varlen = ctx.varlen
        q4, k4, v4 = q, k, v
        do4 = _dense(dout).unsqueeze(0) if varlen else _dense(dout)
        B, S, Hq, D = q4.shape
        args = dict(ctx.args)
        args["cu_seqlens"] = cu_seqlens
        wire = HALO_GRAD_WIRE_DTYPE or q4.dtype

        def grad_pair(shape):
            g = torch.empty((2,) + tuple(shape), dtype=wire, device=q4.device)
            return g

        remote, remote_grads = [], []
        for r in plan.halo_recv:
            hk, hv = rest.pop(0), rest.pop(0)
            g = grad_pair(hk.shape)
            remote.append(K.KVSpan(hk, hv, r.pos_start, dk=g[0], dv=g[1]))
            remote_grads.append(g)
        sink_remote, sink_grads = [], []
        for sr in plan.sink_recv:
            sk, sv = rest.pop(0), rest.pop(0)
            g = grad_pair(sk.shape)
            sink_remote.append(K.KVSpan(sk, sv, sr.pos_start, dk=g[0], dv=g[1]))
            sink_grads.append(g)
        remote = sink_remote + remote

        dq4 = torch.empty_like(q4)
        ws = K.bwd_workspace(q4)
        link = ctx.link
        ops, recvs = [], []   # recvs: (offset, tokens, gradient tensor, (hop, sender) when it sits in a peer slot)
        # With peer stores (a copy-engine put behind an event, no message that the host must post between
        # two calls) the whole backward is ONE call: dK/dV of the received and the local spans in one launch,
        # the received spans' gradients picked up by the side stream while dQ is computed.  Sink gradients
        # travel as messages and many ranks wait for them: with a remote sink the two-call form stays.
        one_call = link is not None and bool(remote) and not sink_remote
        if remote and not one_call:
            with _phase("bwd.halo_spans"):
                K.bwd(q4, remote, out, lse, do4, dq4, workspace=ws, flags=_C.BWD_INIT, **args)
            if link is not None:
                ready = torch.cuda.Event()
                ready.record()
                for r, g in zip(plan.halo_recv, remote_grads):
                    link.put(1, r.hop, r.src, [g], ready)
            else:
                for r, g in zip(plan.halo_recv, remote_grads):
                    ops.append(dist.P2POp(dist.isend, g, ring.global_rank(r.src), ring.group))
            for sr, g in zip(plan.sink_recv, sink_grads):
                ops.append(dist.P2POp(dist.isend, g, ring.global_rank(sr.owner), ring.group))
        for s in plan.halo_send:
            if link is not None:
                g = link.slot_view(1, s.hop, (2, B, s.length) + tuple(k4.shape[2:]), wire)
                recvs.append((S - s.length, s.length, g, (s.hop, s.dst)))
            else:
                g = grad_pair((B, s.length) + tuple(k4.shape[2:]))
                ops.append(dist.P2POp(dist.irecv, g, ring.global_rank(s.dst), ring.group))
                recvs.append((S - s.length, s.length, g, None))
        for s in plan.sink_send:
            g = grad_pair((B, s.n) + tuple(k4.shape[2:]))
            ops.append(dist.P2POp(dist.irecv, g, ring.global_rank(s.dst), ring.group))
            recvs.append((s.offset, s.n, g, None))
        works = _exchange(ops)

        # dK and dV are one stacked tensor, so that K and V parts go through the helper kernels together
        dkv = torch.empty((2,) + tuple(k4.shape), dtype=k4.dtype, device=k4.device)
        dk4, dv4 = dkv[0], dkv[1]
        # Gradients that later ranks return are added in float32 and rounded once.  When they all land
        # on a suffix of the chunk (halo gradients; no sink token inside the chunk), only that suffix is
        # kept in float32: the local K/V go to the kernels as two spans, the body writing its
        # gradients straight into dk/dv, the tail into a small accumulator.
        acc, acc0 = None, 0
        if recvs:
            acc0 = min(r[0] for r in recvs)
            if any(r[0] + r[1] != S for r in recvs) or acc0 <= 0 or len(remote) + 2 > _C.RSWA_MAX_SPANS:
                acc0 = 0
            acc = torch.empty((2, B, S - acc0) + tuple(k4.shape[2:]), dtype=torch.float32, device=k4.device)
            local = [K.KVSpan(k4[:, acc0:], v4[:, acc0:], plan.q_pos_start + acc0, dk=acc[0], dv=acc[1])]
            if acc0 > 0:
                local.insert(0, K.KVSpan(k4[:, :acc0], v4[:, :acc0], plan.q_pos_start, dk=dk4[:, :acc0], dv=dv4[:, :acc0]))
        else:
            local = [K.KVSpan(k4, v4, plan.q_pos_start, dk=dk4, dv=dv4)]
        # second call: dK/dV of the local span, and dQ over every span (the received ones without
        # gradient buffers, their gradients are already on the wire)
        if one_call:
            mid = K.mid_event_for(q4.device)
            with _phase("bwd.local_and_dq"):
                K.bwd(q4, remote + local, out, lse, do4, dq4, workspace=ws, flags=_C.BWD_INIT | _C.BWD_FINISH,
                      mid_event=mid, **args)
            for r, g in zip(plan.halo_recv, remote_grads):
                link.put(1, r.hop, r.src, [g], mid)
        else:
            seen = [K.KVSpan(s.k, s.v, s.pos_start) for s in remote]
            flags = _C.BWD_FINISH | (0 if remote else _C.BWD_INIT)
            with _phase("bwd.local_and_dq"):
                K.bwd(q4, seen + local, out, lse, do4, dq4, workspace=ws, flags=flags, **args)
        with _phase("bwd.grad_wait"):
            _wait(works)
        if acc is not None:
            # [2, B] is one batch axis for the helper kernels (K and V parts in one launch).  The message
            # that covers the whole accumulator (the nearest later rank's) goes last: its addition and the
            # final rounding are one pass.
            L = S - acc0
            flat = lambda t: t.reshape((2 * B,) + tuple(t.shape[2:]))  # noqa: E731  (views: [2, B, ...] is contiguous over [2, B])
            recvs.sort(key=lambda r: r[1])
            # gradients that sit in a peer slot: wait for them to land (in the order they were sent)
            landed = {}
            with _phase("bwd.grad_wait"):
                for r in sorted((r for r in recvs if r[3] is not None), key=lambda r: r[3][0]):
                    landed[r[3]] = link.arrived(1, r[3][0])
            last = recvs[-1] if recvs[-1][0] == acc0 and recvs[-1][1] == L else None
            with _phase("bwd.accumulate"):
                for off, n_tok, g, _slot in (recvs[:-1] if last is not None else recvs):
                    K.halo_accumulate(flat(acc)[:, off - acc0:off - acc0 + n_tok], flat(g))
                if last is not None:
                    K.halo_accumulate_cast(flat(dkv)[:, acc0:], flat(acc), flat(last[2]))
                else:
                    K.cast_from_f32(flat(dkv)[:, acc0:], flat(acc))
            for (hop, sender), n_msg in landed.items():   # the slots have been read: their senders may reuse them
                link.release(1, hop, sender, n_msg)
        if q4.is_cuda:
            K.mirror_status(q4.device)
        if varlen:
            dq4, dk4, dv4 = dq4.squeeze(0), dk4.squeeze(0), dv4.squeeze(0)
        return dq4, dk4, dv4, None, None, None, None, None, None


def ring_ctx(cp_group, cp_size, cp_local_rank, cp_prev_global_rank, cp_next_global_rank, chunk_lens=None) -> RingCtx:
    """Argument defaulting of ring_swa/sliding_window/nonvarlen.py:388-395."""
    if cp_group is None:
        return RingCtx(None, 1, 0, None, None)
    if cp_size is None:
        cp_size = dist.get_world_size(cp_group)
    if cp_local_rank is None:
        cp_local_rank = dist.get_rank(group=cp_group)
    lens = None if chunk_lens is None else tuple(int(x) for x in chunk_lens)
    return RingCtx(cp_group, int(cp_size), int(cp_local_rank), cp_prev_global_rank, cp_next_global_rank, lens)


def attention(q, k, v, window_size: int, n_sink: int, softmax_scale: Optional[float],
              cu_seqlens: Optional[torch.Tensor], cu_host: Optional[Sequence[int]], ring: RingCtx):
    head_dim = q.shape[-1]
    if softmax_scale is None:
        softmax_scale = head_dim ** (-0.5)
    if q.is_cuda and head_dim < K.HEAD_DIM:
        # The kernels are built for a head dimension of 128.  Smaller ones (the reference's own local
        # tests use 64) run on them zero-padded: the padding adds nothing to any score, the padded
        # output and gradient columns are zero and are cut off again -- at the price of the arithmetic
        # and traffic of a 128-wide head.  The scale keeps referring to the caller's head dimension.
        if head_dim % 8:
            raise ValueError(f"head_dim must be a multiple of 8 and at most {K.HEAD_DIM}, got {head_dim}")
        pad = (0, K.HEAD_DIM - head_dim)
        q, k, v = (torch.nn.functional.pad(x, pad) for x in (q, k, v))
        out = RingAttn.apply(q, k, v, int(window_size), int(n_sink), float(softmax_scale), cu_seqlens, cu_host, ring)
        return out[..., :head_dim]
    return RingAttn.apply(q, k, v, int(window_size), int(n_sink), float(softmax_scale), cu_seqlens, cu_host, ring)
