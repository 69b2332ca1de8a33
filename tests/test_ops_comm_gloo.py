"""The communication helpers of ring_swa.ops on gloo CPU ranks, against hand-computed results:
ring_attn_p2p_communicate, broadcast_tensor_to_group, reduce_sum_tesnsor_to_rank,
exchange_and_sum_tensors, get_group_local_to_global_rank_map (ring_swa/ops/comm.py:8-232 of the
reference).  Four ranks; where it matters that group-local and global ranks differ the group under test
is the sub-group of global ranks (1, 2, 3) (torch orders a group's ranks ascending)."""
import json
import os
import sys
import tempfile

import pytest
import torch
import torch.multiprocessing as mp

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)


def _rank_body(rank, ws, port, outdir):
    for p in (ROOT, os.path.join(ROOT, "ring-sliding-window-attention_b200"), HERE):
        if p not in sys.path:
            sys.path.insert(0, p)
    import torch.distributed as dist
    from datetime import timedelta
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.set_num_threads(1)
    dist.init_process_group("gloo", rank=rank, world_size=ws, timeout=timedelta(seconds=120))
    from ring_swa.ops import (broadcast_tensor_to_group, exchange_and_sum_tensors, get_group_local_to_global_rank_map,
                              reduce_sum_tesnsor_to_rank, ring_attn_p2p_communicate)
    res = {}
    world = dist.group.WORLD
    # -- rank map: identity on the world group, the listed order on a sub-group (every rank creates the group)
    sub_ranks = [1, 2, 3]
    sub = dist.new_group(ranks=sub_ranks)
    res["map_world"] = get_group_local_to_global_rank_map(world)
    res["map_none"] = get_group_local_to_global_rank_map(None)
    if rank in sub_ranks:
        res["map_sub"] = get_group_local_to_global_rank_map(sub)
        res["map_sub_again_is_cached"] = get_group_local_to_global_rank_map(sub) is get_group_local_to_global_rank_map(sub)
    # -- one ring step: send to the next rank, receive from the previous one
    send = torch.full((3, 2), float(rank + 1))
    recv = torch.zeros(3, 2)
    reqs = ring_attn_p2p_communicate(rank, send, (rank + 1) % ws, recv, (rank - 1) % ws, world)
    assert len(reqs) == 2
    for r in reqs:
        r.wait()
    res["p2p_recv"] = recv[0, 0].item()
    # -- broadcast from global rank 2, asynchronous handle
    t = torch.arange(4, dtype=torch.float32) * (10 if rank == 2 else -1)
    work = broadcast_tensor_to_group(t, 2, world)
    work.wait()
    res["bcast"] = t.tolist()
    # -- sum-reduce to global rank 1 (the result is only defined there)
    t = torch.full((2, 2), float(rank + 1))
    out = reduce_sum_tesnsor_to_rank(t, 1, world)
    res["reduce_same_tensor"] = out is t
    res["reduce"] = out[0, 0].item()
    # -- personalised exchange: ranks 0 and 3 send to rank 1, rank 1 to rank 0, rank 2 to itself
    dst = {0: 1, 1: 0, 2: 2, 3: 1}[rank]
    got = exchange_and_sum_tensors(torch.full((2,), float(10 ** rank)), dst, world)
    res["exchange"] = got.tolist()
    # ... and inside the sub-group, where send_to_rank is a group-local rank
    if rank in sub_ranks:
        me = sub_ranks.index(rank)                 # group-local rank
        got = exchange_and_sum_tensors(torch.full((1,), float(me + 1)), (me + 1) % 3, sub)
        res["exchange_sub"] = got.item()
    with open(os.path.join(outdir, f"r{rank}.json"), "w") as f:
        json.dump(res, f)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.timeout(300)
def test_comm_helpers_on_four_gloo_ranks():
    ws = 4
    with tempfile.TemporaryDirectory() as tmp:
        mp.spawn(_rank_body, args=(ws, 29771, tmp), nprocs=ws, join=True)
        res = [json.load(open(os.path.join(tmp, f"r{r}.json"))) for r in range(ws)]
    for r in range(ws):
        assert res[r]["map_world"] == {str(i): i for i in range(ws)}
        assert res[r]["map_none"] == {}
        assert res[r]["p2p_recv"] == float((r - 1) % ws + 1)            # what the previous rank sent
        assert res[r]["bcast"] == [0.0, 10.0, 20.0, 30.0]
        assert res[r]["reduce_same_tensor"] is True
    assert res[1]["reduce"] == 1.0 + 2.0 + 3.0 + 4.0
    # group-local rank i of the sub-group is global rank i + 1
    for r in (1, 2, 3):
        assert res[r]["map_sub"] == {"0": 1, "1": 2, "2": 3}
        assert res[r]["map_sub_again_is_cached"] is True
    assert "map_sub" not in res[0]
    assert res[0]["exchange"] == [10.0, 10.0]            # from rank 1
    assert res[1]["exchange"] == [1001.0, 1001.0]        # from ranks 0 and 3
    assert res[2]["exchange"] == [100.0, 100.0]          # from itself
    assert res[3]["exchange"] == [0.0, 0.0]              # nobody sent
    # sub-group ring: group-local i sends the value i + 1 to group-local i + 1 (mod 3); global ranks (1, 2, 3) are local (0, 1, 2)
    assert res[1]["exchange_sub"] == 3.0 and res[2]["exchange_sub"] == 1.0 and res[3]["exchange_sub"] == 2.0
