"""Single-GPU StreamingLLM attention under the reference's names (ring_swa/streaming_llm/naive.py:213-237).

The reference builds these from two flash-attn calls and a merge; here they are the cp_group=None case of
the ring functions (one kernel pass with the sink folded in as an extra key block).
"""
from typing import Optional

import torch

from .nonvarlen import ring_streaming_llm_attn
from .varlen import ring_streaming_llm_attn_varlen


def naive_streaming_llm_attn(q, k, v, window_size: int, softmax_scale: Optional[float] = None):
    return ring_streaming_llm_attn(q, k, v, window_size, softmax_scale=softmax_scale)


def naive_streaming_llm_attn_varlen(q, k, v, window_size: int, cu_seqlens: torch.Tensor,
                                    softmax_scale: Optional[float] = None):
    return ring_streaming_llm_attn_varlen(q, k, v, window_size, cu_seqlens, cp_size=1,
                                          softmax_scale=softmax_scale)


class StreamingLLMAttn:
    """The reference's single-GPU autograd class by name (ring_swa/streaming_llm/naive.py:11-20):
    apply(q, k, v, window_size, softmax_scale)."""

    @staticmethod
    def apply(q, k, v, window_size, softmax_scale=None):
        return naive_streaming_llm_attn(q, k, v, window_size, softmax_scale)


class StreamingLLMAttnVarlen:
    """ring_swa/streaming_llm/naive.py:90-100: apply(q, k, v, window_size, cu_seqlens, softmax_scale)."""

    @staticmethod
    def apply(q, k, v, window_size, cu_seqlens, softmax_scale=None):
        return naive_streaming_llm_attn_varlen(q, k, v, window_size, cu_seqlens, softmax_scale)
