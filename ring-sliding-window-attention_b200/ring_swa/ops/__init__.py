"""Operator-level names of the reference's ring_swa.ops that remain meaningful here
(ring_swa/ops/__init__.py:1-38).  The flash-attn wrappers have no counterpart: the attention
arithmetic lives in librswa.so and is reached through ring_swa._kernels."""
from .comm import (
    ring_attn_p2p_communicate,
    broadcast_tensor_to_group,
    reduce_sum_tesnsor_to_rank,
    exchange_and_sum_tensors,
    get_group_local_to_global_rank_map,
)
from .merge import merge_attn_out

__all__ = [
    "ring_attn_p2p_communicate",
    "broadcast_tensor_to_group",
    "reduce_sum_tesnsor_to_rank",
    "exchange_and_sum_tensors",
    "merge_attn_out",
    "get_group_local_to_global_rank_map",
]
