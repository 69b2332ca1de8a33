"""Peer-store exchange of halo K/V (forward) and halo gradients (backward) between the GPUs of one node.

What the reference does with one NCCL isend / irecv pair per hop (ring_swa/ops/comm.py:8-40) is done here
without any communication kernel on the SMs: every rank owns a receive buffer in symmetric memory (mapped
into all peers), a sender moves its message into the receiver's buffer with a copy-engine transfer
followed by a one-word flag, and the receiver puts a one-thread wait for that flag on its compute stream
in front of the first kernel that needs the data.  The attention kernels then read the landed tiles from
LOCAL memory with their ordinary TMA loads; nothing loads from a peer and nothing uses multicast.

Protocol, per pair (src, dst = src + hop) and direction, with sequence numbers that only grow:
  sender    wait ack >= n - 1 (the slot is free)  ->  put message into dst's slot  ->  dst.data_flag = n
  receiver  wait data_flag >= n  ->  read the slot (copy out / accumulate)  ->  src.ack_flag = n
All waits are bounded (rswa_flag_wait): if a number does not arrive in time the device status word is
raised and the next call of the public API reports it, instead of a hung stream.

Only the attention functions' own halo traffic goes this way; sink tokens (a few hundred bytes, only in
the StreamingLLM functions) keep torch.distributed point-to-point messages.
"""
from __future__ import annotations

import os
from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

from . import _kernels as K

MAX_HOPS = 8
_FLAG_BYTES = 4096          # 1024 int32 words at the head of every rank's buffer
# flag word indices (per hop h in 1..MAX_HOPS): data arriving / acknowledgement coming back, forward / backward
_DATA_F, _ACK_F, _DATA_B, _ACK_B = 0, 16, 32, 48

WAIT_TIMEOUT_S = float(os.environ.get("RING_SWA_PEER_TIMEOUT_S", "10"))


def wanted() -> bool:
    """Peer stores are the default between GPUs; RING_SWA_HALO=nccl keeps the point-to-point messages."""
    return os.environ.get("RING_SWA_HALO", "peer").lower() != "nccl"


def _align(n: int, a: int = 256) -> int:
    return (n + a - 1) // a * a


class PeerLink:
    """One rank's end of the exchange for one (process group, buffer layout)."""

    def __init__(self, group, device: torch.device, slot_bytes: List[int]):
        import torch.distributed._symmetric_memory as symm_mem
        self.group, self.device = group, device
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        # layout: flags | forward slots (hop 1..) | backward slots (hop 1..)
        self.slot_bytes = list(slot_bytes)
        offs, off = [], _FLAG_BYTES
        for _direction in range(2):
            row = []
            for nb in slot_bytes:
                row.append(off)
                off += _align(nb)
            offs.append(row)
        self.offsets, self.nbytes = offs, off
        try:
            symm_mem.enable_symm_mem_for_group(group.group_name)
        except Exception:
            pass                                   # newer torch needs no registration
        self.buf = symm_mem.empty(self.nbytes, dtype=torch.uint8, device=device)
        self.hdl = symm_mem.rendezvous(self.buf, group)
        self.ptrs = [int(p) for p in self.hdl.buffer_ptrs]       # this buffer in every rank, by group rank
        self.buf[:_FLAG_BYTES].zero_()
        torch.cuda.current_stream(device).synchronize()
        dist.barrier(group)                                          # nobody writes a flag that is zeroed afterwards
        self.side = torch.cuda.Stream(device=device)
        self.sent = {}    # (direction, hop) -> messages put so far
        self.recvd = {}   # (direction, hop) -> messages consumed so far

    # -- addresses
    def flag_ptr(self, rank: int, base: int, hop: int) -> int:
        return self.ptrs[rank] + 4 * (base + hop)

    def slot_ptr(self, rank: int, direction: int, hop: int) -> int:
        return self.ptrs[rank] + self.offsets[direction][hop - 1]

    def slot_view(self, direction: int, hop: int, shape, dtype) -> torch.Tensor:
        """This rank's own slot as a tensor (local memory)."""
        n = 1
        for s in shape:
            n *= s
        nb = n * torch.empty((), dtype=dtype).element_size()
        off = self.offsets[direction][hop - 1]
        return self.buf[off:off + nb].view(dtype).view(shape)

    # -- protocol
    def put(self, direction: int, hop: int, dst: int, parts: List[torch.Tensor], ready) -> None:
        """Move `parts` (tensors whose rows per leading index are contiguous; laid out one after the other
        in the slot) into dst's slot for (direction, hop), on the side stream, behind `ready` (a
        torch.cuda.Event, or the raw handle of an event of the kernel library)."""
        key = (direction, hop)
        n = self.sent.get(key, 0) + 1
        self.sent[key] = n
        data_base, ack_base = (_DATA_F, _ACK_F) if direction == 0 else (_DATA_B, _ACK_B)
        with torch.cuda.stream(self.side):
            if isinstance(ready, int):
                K.stream_wait_event(self.side, ready)
            else:
                self.side.wait_event(ready)
            if n > 1:   # the receiver has read message n - 1 out of the slot
                K.flag_wait(self.flag_ptr(self.rank, ack_base, hop), n - 1, self.device, WAIT_TIMEOUT_S)
            base = self.slot_ptr(dst, direction, hop)
            off = 0
            for i, t in enumerate(parts):
                rows = t.shape[0]
                row_bytes = t[0].numel() * t.element_size()
                last = i + 1 == len(parts)
                K.peer_put(base + off, row_bytes, t, self.flag_ptr(dst, data_base, hop) if last else 0, n)
                t.record_stream(self.side)
                off += rows * row_bytes

    def arrived(self, direction: int, hop: int) -> int:
        """Queues the wait for the next message of (direction, hop) on the current stream; returns its number."""
        key = (direction, hop)
        n = self.recvd.get(key, 0) + 1
        self.recvd[key] = n
        base = _DATA_F if direction == 0 else _DATA_B
        K.flag_wait(self.flag_ptr(self.rank, base, hop), n, self.device, WAIT_TIMEOUT_S)
        return n

    def release(self, direction: int, hop: int, src: int, n: int) -> None:
        """Tells src, on the current stream, that message n has been read out of the slot."""
        base = _ACK_F if direction == 0 else _ACK_B
        K.flag_set(self.flag_ptr(src, base, hop), n)


_links: Dict[Tuple, PeerLink] = {}


def slot_bytes_for(cp: int, S: int, W: int, batch: int, hkv: int, head_dim: int,
                   S_min: Optional[int] = None) -> Optional[List[int]]:
    """Bytes of the receive slot of every hop (float32 gradients included) for a geometry, or None when
    nothing travels or the window reaches over more chunks than there are flag words for.  `S` is the
    largest chunk of the group and `S_min` the smallest where they differ: a message holds at most S
    tokens, and the window reaches over at most ceil(W / S_min) chunks."""
    S_min = S if S_min is None else S_min
    hops = min((W + S_min - 1) // S_min, cp - 1)
    if hops < 1 or hops > MAX_HOPS:
        return None
    return [2 * batch * min(S, max(0, W - (h - 1) * S_min)) * hkv * head_dim * 4 for h in range(1, hops + 1)]


def link_for(group, device: torch.device, cp: int, S: int, W: int, batch: int, hkv: int, head_dim: int,
             S_min: Optional[int] = None) -> Optional[PeerLink]:
    """The link of this (group, device), its slots large enough for every halo message of the geometry
    (slot_bytes_for).  Every rank of the group must call this with the same arguments, the first time and
    whenever a larger geometry shows up (a collective set-up)."""
    need = slot_bytes_for(cp, S, W, batch, hkv, head_dim, S_min)
    if need is None:
        return None
    key = (id(group), device.index)
    link = _links.get(key)
    if link is not None and len(link.slot_bytes) >= len(need) and all(a >= b for a, b in zip(link.slot_bytes, need)):
        return link
    if link is not None:   # grow: every rank sees the same geometry, so every rank gets here together
        need = [max(a, b) for a, b in zip(need + [0] * len(link.slot_bytes), link.slot_bytes + [0] * len(need))]
        need = [x for x in need if x > 0]
        torch.cuda.synchronize(device)
        dist.barrier(group)
    link = PeerLink(group, device, need)
    _links[key] = link
    return link
