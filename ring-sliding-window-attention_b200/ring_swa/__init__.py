"""ring_swa -- ring sliding-window / StreamingLLM attention on B200 (sm_100a).

Same public functions and argument meaning as the reference package of this name
(ring_swa/__init__.py:1-9): hand-written CUDA kernels behind a C ABI instead of flash-attn + Triton.
"""
from .sliding_window import ring_sliding_window_attn, ring_sliding_window_attn_varlen
from .streaming_llm import ring_streaming_llm_attn, ring_streaming_llm_attn_varlen

__all__ = [
    "ring_sliding_window_attn",
    "ring_sliding_window_attn_varlen",
    "ring_streaming_llm_attn",
    "ring_streaming_llm_attn_varlen",
]
