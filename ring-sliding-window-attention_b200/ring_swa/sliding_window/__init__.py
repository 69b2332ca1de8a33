from .nonvarlen import ring_sliding_window_attn
from .varlen import ring_sliding_window_attn_varlen

__all__ = ["ring_sliding_window_attn", "ring_sliding_window_attn_varlen"]
