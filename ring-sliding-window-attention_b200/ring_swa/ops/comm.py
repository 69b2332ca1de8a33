"""Communication helpers under the reference's names (ring_swa/ops/comm.py).

The attention functions of this package plan their own halo exchange (ring_swa/_plan.py) and do not
call these; they are kept for code written against ring_swa.ops.
"""
import os
from typing import Dict, List, Tuple

import torch
import torch.distributed as dist
from torch.distributed import ProcessGroup


def ring_attn_p2p_communicate(rank: int, send_tensor: torch.Tensor, send_rank: int, recv_tensor: torch.Tensor,
                              recv_rank: int, cp_group: ProcessGroup) -> List:
    """One send to `send_rank` and one receive from `recv_rank` (global ranks); returns the requests.
    Even ranks send first, odd ranks receive first (ring_swa/ops/comm.py:8-40)."""
    reqs = []
    if rank % 2 == 0:
        reqs.append(dist.isend(send_tensor, send_rank, cp_group))
        reqs.append(dist.irecv(recv_tensor, recv_rank, cp_group))
    else:
        reqs.append(dist.irecv(recv_tensor, recv_rank, cp_group))
        reqs.append(dist.isend(send_tensor, send_rank, cp_group))
    return reqs


def broadcast_tensor_to_group(tensor: torch.Tensor, src_rank: int, cp_group: ProcessGroup):
    """Asynchronous broadcast from global rank `src_rank` (ring_swa/ops/comm.py:43-69)."""
    return dist.broadcast(tensor, src=src_rank, group=cp_group, async_op=True)


def reduce_sum_tesnsor_to_rank(tensor: torch.Tensor, dst_rank: int, cp_group: ProcessGroup) -> torch.Tensor:
    """In-place sum-reduce to global rank `dst_rank`, waited for (ring_swa/ops/comm.py:72-99; the
    spelling of the name is the reference's)."""
    work = dist.reduce(tensor, dst=dst_rank, op=dist.ReduceOp.SUM, group=cp_group, async_op=True)
    work.wait()
    return tensor


def exchange_and_sum_tensors(tensor_to_send: torch.Tensor, send_to_rank: int, cp_group: ProcessGroup) -> torch.Tensor:
    """Every rank sends one tensor to one group rank; returns the sum of what this rank received
    (ring_swa/ops/comm.py:102-149).  Built on all_gather so that it also runs on backends without
    all_to_all.  Cost: two all_gathers (the destinations, then every rank's tensor: world_size times the
    bytes of the reference's single all_to_all, which moves one tensor per rank pair) and a local sum;
    meant for the few hundred bytes of sink gradients the reference uses it for, not for bulk data."""
    ws = dist.get_world_size(group=cp_group)
    me = dist.get_rank(group=cp_group)
    dst = torch.tensor([int(send_to_rank)], dtype=torch.long, device=tensor_to_send.device)
    dsts = [torch.empty_like(dst) for _ in range(ws)]
    bufs = [torch.empty_like(tensor_to_send) for _ in range(ws)]
    dist.all_gather(dsts, dst, group=cp_group)
    dist.all_gather(bufs, tensor_to_send.contiguous(), group=cp_group)
    out = torch.zeros_like(tensor_to_send)
    for r, d in enumerate(torch.cat(dsts).tolist()):
        if d == me:
            out += bufs[r]
    return out


_rank_map_cache: Dict[Tuple[int, ...], Dict[int, int]] = {}


def get_group_local_to_global_rank_map(group: ProcessGroup) -> Dict[int, int]:
    """{group-local rank: global rank} for `group` (ring_swa/ops/comm.py:152-232).

    The reference all_gathers the pairs; torch.distributed already knows them, so no collective is
    needed, but the result (and the cache per set of ranks) is the same."""
    if group is None:
        return {}
    ranks = tuple(dist.get_process_group_ranks(group))
    if ranks not in _rank_map_cache:
        _rank_map_cache[ranks] = {i: g for i, g in enumerate(ranks)}
    return _rank_map_cache[ranks]
