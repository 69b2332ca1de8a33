"""merge_attn_out: in-place log-sum-exp merge, the signature of ring_swa/ops/merge.py:150-155."""
import torch

from .. import _kernels as K


def merge_attn_out(attn_out: torch.Tensor, softmax_lse: torch.Tensor, new_attn_out: torch.Tensor,
                   new_softmax_lse: torch.Tensor) -> None:
    """Folds (new_attn_out, new_softmax_lse) into (attn_out, softmax_lse) in place.

    attn_out / new_attn_out: [batch, seq_len, heads, 128] bf16 or fp16; softmax_lse / new_softmax_lse:
    [batch, heads, seq_len] float32.  Runs the vectorised CUDA merge kernel; a pair of -inf merges to
    (0, -inf) instead of the NaN the formula of ring_swa/ops/merge.py:138-147 would give.
    """
    if attn_out.dtype not in (torch.bfloat16, torch.float16) or new_attn_out.dtype != attn_out.dtype:
        raise ValueError("merge_attn_out: both outputs must be bfloat16 or float16 and of one dtype")
    if softmax_lse.dtype != torch.float32:
        raise ValueError("merge_attn_out: softmax_lse must be float32 (it is updated in place)")
    if new_softmax_lse.dtype != torch.float32 or new_softmax_lse.stride() != softmax_lse.stride():
        new_softmax_lse = new_softmax_lse.to(torch.float32).contiguous()
        if new_softmax_lse.stride() != softmax_lse.stride():
            raise ValueError("merge_attn_out: the two lse tensors must share their layout")
    K.merge(attn_out, softmax_lse, new_attn_out, new_softmax_lse)
