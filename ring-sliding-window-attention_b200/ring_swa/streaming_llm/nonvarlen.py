"""ring_streaming_llm_attn: same signature as ring_swa/streaming_llm/nonvarlen.py:400-411."""
from typing import Optional

import torch
from torch.distributed import ProcessGroup

from .._ring import attention, ring_ctx
from ..sliding_window.nonvarlen import _check_nonvarlen


def ring_streaming_llm_attn(
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
    *,
    num_sink_tokens: int = 1,
):
    """Ring StreamingLLM attention: the sliding window plus the sink at the start of the sequence.

    Arguments as in ring_sliding_window_attn.  Every query additionally attends to the first
    `num_sink_tokens` tokens of its sequence; the default of one is what the reference computes
    (ring_swa/streaming_llm/nonvarlen.py:48-51), the keyword is an extension.  Each batch row uses its
    own first token (the reference takes batch row 0's for every row, which is the same under its
    stated assumption that all sinks are identical).
    """
    _check_nonvarlen(q, k, v)
    ring = ring_ctx(cp_group, cp_size, cp_local_rank, cp_prev_global_rank, cp_next_global_rank)
    return attention(q, k, v, window_size, num_sink_tokens, softmax_scale, None, None, ring)


class RingStreamingLLMAttn:
    """The reference's autograd class by name (ring_swa/streaming_llm/nonvarlen.py:20-35): `apply` takes
    its forward's positional arguments in its order (one sink token); `cp_stream` is accepted and not used."""

    @staticmethod
    def apply(q, k, v, window_size, cp_group, cp_size, cp_local_rank, cp_prev_global_rank,
              cp_next_global_rank, cp_stream=None, softmax_scale=None):
        return ring_streaming_llm_attn(q, k, v, window_size, cp_group, cp_size, cp_local_rank,
                                       cp_prev_global_rank, cp_next_global_rank, softmax_scale)
