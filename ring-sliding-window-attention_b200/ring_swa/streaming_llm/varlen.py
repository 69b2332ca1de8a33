"""ring_streaming_llm_attn_varlen: same signature as ring_swa/streaming_llm/varlen.py:476-488."""
from typing import Optional, Sequence

import torch
from torch.distributed import ProcessGroup

from .._ring import attention, ring_ctx
from ..sliding_window.varlen import _varlen_prologue


def ring_streaming_llm_attn_varlen(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    window_size: int,
    cu_seqlens: torch.Tensor,
    cp_group: Optional[ProcessGroup] = None,
    cp_size: Optional[int] = None,
    cp_local_rank: Optional[int] = None,
    cp_prev_global_rank: Optional[int] = None,
    cp_next_global_rank: Optional[int] = None,
    softmax_scale: Optional[float] = None,
    *,
    num_sink_tokens: int = 1,
    cp_chunk_lens: Optional[Sequence[int]] = None,
) -> torch.Tensor:
    """Ring StreamingLLM attention over packed variable-length sequences.

    Arguments as in ring_sliding_window_attn_varlen.  Every query additionally attends to the first
    `num_sink_tokens` tokens of its OWN sequence.  The reference attends to global token 0 instead and
    documents the assumption that every sequence starts with the same sink content
    (ring_swa/streaming_llm/varlen.py:50-63, 476-488); under that assumption both are the same function,
    and the sink gradient lands on each sequence's own first token as in the reference (:454-467).
    `cp_chunk_lens`: chunks of different lengths per rank, as in ring_sliding_window_attn_varlen.
    """
    cu_seqlens, cu_host = _varlen_prologue(q, k, v, cu_seqlens, cp_size, cp_chunk_lens)
    ring = ring_ctx(cp_group, cp_size, cp_local_rank, cp_prev_global_rank, cp_next_global_rank, cp_chunk_lens)
    return attention(q, k, v, window_size, num_sink_tokens, softmax_scale, cu_seqlens, cu_host, ring)


class RingStreamingLLMVarlen:
    """The reference's autograd class by name (ring_swa/streaming_llm/varlen.py:20-37): `apply` takes its
    forward's positional arguments in its order (one sink token); `max_seqlen` and `cp_stream` are
    accepted and not used."""

    @staticmethod
    def apply(q, k, v, window_size, cu_seqlens, max_seqlen, cp_group, cp_size, cp_local_rank,
              cp_prev_global_rank, cp_next_global_rank, cp_stream=None, softmax_scale=None):
        return ring_streaming_llm_attn_varlen(q, k, v, window_size, cu_seqlens, cp_group, cp_size, cp_local_rank,
                                              cp_prev_global_rank, cp_next_global_rank, softmax_scale)
