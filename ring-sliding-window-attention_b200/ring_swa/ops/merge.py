"""merge_attn_out: in-place log-sum-exp merge, the signature of ring_swa/ops/merge.py:150-155."""
import torch

from .. import _kernels as K


def merge_attn_out(attn_out: torch.Tensor, softmax_lse: torch.Tensor, new_attn_out: torch.Tensor,
                   new_softmax_lse: torch.Tensor) -> None:
    """Folds (new_attn_out, new_softmax_lse) into (attn_out, softmax_lse) in place.

    attn_out / new_attn_out: [batch, seq_len, heads, head_dim]; softmax_lse / new_softmax_lse:
    [batch, heads, seq_len].  Two dtype combinations run, each on its own CUDA kernel:
      * the reference's accumulators (ring_swa/sliding_window/nonvarlen.py:60-75): attn_out float32 (strided
        views allowed), softmax_lse float32 or float64, new_attn_out bf16/fp16/float32;
      * attn_out and new_attn_out both bf16 or fp16 with a float32 softmax_lse (head_dim 128).
    A pair of -inf merges to (0, -inf) instead of the NaN the formula of ring_swa/ops/merge.py:138-147
    would give.  There is no torch fallback: without the CUDA library this raises.
    """
    if new_softmax_lse.dtype != torch.float32:
        new_softmax_lse = new_softmax_lse.to(torch.float32)
    if new_softmax_lse.stride(-1) != 1:
        new_softmax_lse = new_softmax_lse.contiguous()
    if attn_out.dtype == torch.float32:
        K.merge_acc(attn_out, softmax_lse, new_attn_out, new_softmax_lse)
        return
    if attn_out.dtype not in (torch.bfloat16, torch.float16) or new_attn_out.dtype != attn_out.dtype:
        raise ValueError("merge_attn_out: attn_out must be float32, or both outputs bfloat16 / float16 of one dtype")
    if softmax_lse.dtype != torch.float32:
        raise ValueError("merge_attn_out: with a 16-bit attn_out softmax_lse must be float32 (it is updated in place)")
    if new_softmax_lse.stride() != softmax_lse.stride():
        new_softmax_lse = new_softmax_lse.contiguous()
        if new_softmax_lse.stride() != softmax_lse.stride():
            raise ValueError("merge_attn_out: the two lse tensors must share their layout")
    K.merge(attn_out, softmax_lse, new_attn_out, new_softmax_lse)


# The reference binds merge_attn_out to its Triton kernel wrapper of this name where Triton >= 3 is present
# (ring_swa/ops/merge.py:150, 196-200); code that imports that name gets the CUDA kernels here.  Its pure
# torch variant (torch_merge_attn_out, :16-66) has no counterpart: there is no path without the library.
triton_merge_attn_out = merge_attn_out
