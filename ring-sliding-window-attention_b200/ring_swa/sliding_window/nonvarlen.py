"""ring_sliding_window_attn: same signature as ring_swa/sliding_window/nonvarlen.py:341-352."""
from typing import Optional

import torch
from torch.distributed import ProcessGroup

from .._ring import attention, ring_ctx


def _check_nonvarlen(q, k, v):
    # the reference's asserts, ring_swa/sliding_window/nonvarlen.py:36-41
    assert q.dim() == 4 and k.dim() == 4 and v.dim() == 4, "q, k, v must be [batch, seq_len, heads, head_dim]"
    assert q.shape[1] == k.shape[1] == v.shape[1], "Sequence length must be the same"
    assert q.shape[2] % k.shape[2] == 0, "Number of query heads must be divisible by number of key/value heads"


def ring_sliding_window_attn(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    window_size: int,
    cp_group: Optional[ProcessGroup] = None,
    cp_size: Optional[int] = None,
    cp_local_rank: Optional[int] = None,
    cp_prev_global_rank: Optional[int] = None,
    cp_next_global_rank: Optional[int] = None,
    softmax_scale: Optional[float] = None,
):
    """Ring sliding window attention without variable length.

    q [batch, seq_len, num_q_heads, head_dim]; k, v [batch, seq_len, num_kv_heads, head_dim]: this rank's
    chunk of the sequence (chunk i lives on group rank i).  Each query attends to itself and the
    `window_size` previous tokens.  With cp_group=None the whole sequence is on this GPU.  cp_size,
    cp_local_rank and the previous/next global ranks default as in the reference
    (ring_swa/sliding_window/nonvarlen.py:388-395).  Returns [batch, seq_len, num_q_heads, head_dim].
    """
    _check_nonvarlen(q, k, v)
    ring = ring_ctx(cp_group, cp_size, cp_local_rank, cp_prev_global_rank, cp_next_global_rank)
    return attention(q, k, v, window_size, 0, softmax_scale, None, None, ring)


class RingSlidingWindowAttn:
    """The reference's autograd class by name (ring_swa/sliding_window/nonvarlen.py:17-32): `apply` takes
    its forward's positional arguments in its order.  `cp_stream` is accepted and not used (the halo
    exchange runs on a stream of its own); differentiation goes through the one autograd function
    behind ring_sliding_window_attn."""

    @staticmethod
    def apply(q, k, v, window_size, cp_group, cp_size, cp_local_rank, cp_prev_global_rank,
              cp_next_global_rank, cp_stream=None, softmax_scale=None):
        return ring_sliding_window_attn(q, k, v, window_size, cp_group, cp_size, cp_local_rank,
                                        cp_prev_global_rank, cp_next_global_rank, softmax_scale)
