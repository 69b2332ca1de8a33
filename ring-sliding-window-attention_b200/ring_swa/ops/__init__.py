"""Operator-level names of the reference's ring_swa.ops (ring_swa/ops/__init__.py:1-38), all backed by
librswa.so: the communication helpers, the four attention operators that stand where the
reference calls flash-attn, the attention-plus-merge steps built on them, and the merge itself."""
from .comm import (
    ring_attn_p2p_communicate,
    broadcast_tensor_to_group,
    reduce_sum_tesnsor_to_rank,
    exchange_and_sum_tensors,
    get_group_local_to_global_rank_map,
)
from .wrap_flash import (
    wrapped_flash_attn_fwd,
    wrapped_flash_attn_fwd_varlen,
    wrapped_flash_attn_bwd,
    wrapped_flash_attn_bwd_varlen,
)
from .attn import (
    flash_attn_fwd_func,
    flash_attn_bwd_func,
    flash_attn_varlen_fwd_func,
    flash_attn_varlen_bwd_func,
)
from .merge import merge_attn_out

__all__ = [
    "ring_attn_p2p_communicate",
    "broadcast_tensor_to_group",
    "reduce_sum_tesnsor_to_rank",
    "exchange_and_sum_tensors",
    "wrapped_flash_attn_fwd",
    "wrapped_flash_attn_fwd_varlen",
    "wrapped_flash_attn_bwd",
    "wrapped_flash_attn_bwd_varlen",
    "flash_attn_fwd_func",
    "flash_attn_bwd_func",
    "flash_attn_varlen_fwd_func",
    "flash_attn_varlen_bwd_func",
    "merge_attn_out",
    "get_group_local_to_global_rank_map",
]
