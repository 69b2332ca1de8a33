from .nonvarlen import ring_streaming_llm_attn
from .varlen import ring_streaming_llm_attn_varlen

__all__ = ["ring_streaming_llm_attn", "ring_streaming_llm_attn_varlen"]
