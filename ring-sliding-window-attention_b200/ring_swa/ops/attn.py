"""Attention-plus-merge steps under the reference's names (ring_swa/ops/attn.py:12-196).

Each forward function computes one partial result over the given keys and folds it into the
caller's running (global_attn_out, global_softmax_lse); each backward function writes dq and the
stacked dkv for the same keys from the final out / lse.  kv and dkv are stacked [2, B, S, Hkv, D].

A call with more queries than keys keeps the reference's meaning unless it is plain full attention
(ring_swa/ops/attn.py:21, 38-60, 93-126; the same predicate, `causal` included): the leading
q_len - kv_len queries see every key, the trailing kv_len queries see the window, both parts with
causal=False; these are two launches on disjoint query rows, and dkv is the float32 sum of the two
parts.  The backward differentiates exactly that (the reference hands `causal` on to the parts of its
backward, which for causal=True is not the gradient of its own forward; its callers only take this
path with causal=False).  Sliced lse views are passed as they are (the kernels take a batch and a
head stride), so the reference's defensive .clone() calls have no counterpart.
"""
from typing import Tuple

import torch

from .merge import merge_attn_out
from .wrap_flash import (
    wrapped_flash_attn_bwd,
    wrapped_flash_attn_bwd_varlen,
    wrapped_flash_attn_fwd,
    wrapped_flash_attn_fwd_varlen,
)


def flash_attn_fwd_func(q: torch.Tensor, kv: torch.Tensor, softmax_scale: float, window_size: Tuple[int, int],
                        causal: bool, global_attn_out: torch.Tensor, global_softmax_lse: torch.Tensor) -> None:
    if not (q.shape[1] <= kv.shape[2] or (not causal and tuple(window_size) == (-1, -1))):
        kv_len = kv.shape[2]
        flash_attn_fwd_func(q[:, :-kv_len], kv, softmax_scale, (-1, -1), False,
                            global_attn_out[:, :-kv_len], global_softmax_lse[:, :, :-kv_len])
        flash_attn_fwd_func(q[:, -kv_len:], kv, softmax_scale, window_size, False,
                            global_attn_out[:, -kv_len:], global_softmax_lse[:, :, -kv_len:])
        return
    out, lse = wrapped_flash_attn_fwd(q=q, k=kv[0], v=kv[1], softmax_scale=softmax_scale, causal=causal,
                                      window_size=window_size)
    merge_attn_out(global_attn_out, global_softmax_lse, out, lse)


def flash_attn_bwd_func(q: torch.Tensor, kv: torch.Tensor, o: torch.Tensor, softmax_lse: torch.Tensor,
                        do: torch.Tensor, dq: torch.Tensor, dkv: torch.Tensor, softmax_scale: float,
                        window_size: Tuple[int, int], causal: bool) -> None:
    if not (q.shape[1] <= kv.shape[2] or (not causal and tuple(window_size) == (-1, -1))):
        kv_len = kv.shape[2]
        acc = torch.zeros_like(dkv, dtype=torch.float32)
        part = torch.empty_like(acc)
        flash_attn_bwd_func(q[:, :-kv_len], kv, o[:, :-kv_len], softmax_lse[:, :, :-kv_len], do[:, :-kv_len],
                            dq[:, :-kv_len], part, softmax_scale, (-1, -1), False)
        acc.add_(part)
        flash_attn_bwd_func(q[:, -kv_len:], kv, o[:, -kv_len:], softmax_lse[:, :, -kv_len:], do[:, -kv_len:],
                            dq[:, -kv_len:], part, softmax_scale, window_size, False)
        acc.add_(part)
        dkv.copy_(acc)
        return
    wrapped_flash_attn_bwd(q=q, k=kv[0], v=kv[1], o=o, softmax_lse=softmax_lse, do=do, dq=dq, dk=dkv[0],
                           dv=dkv[1], softmax_scale=softmax_scale, window_size=window_size, causal=causal)


def flash_attn_varlen_fwd_func(q: torch.Tensor, kv: torch.Tensor, softmax_scale: float,
                               window_size: Tuple[int, int], cu_seqlens_q: torch.Tensor,
                               cu_seqlens_k: torch.Tensor, max_seqlen_q, max_seqlen_k, causal: bool,
                               global_attn_out: torch.Tensor, global_softmax_lse: torch.Tensor) -> None:
    """q [1,T,Hq,D], kv [2,1,T,Hkv,D]; the accumulators keep their leading batch of 1."""
    out, lse = wrapped_flash_attn_fwd_varlen(
        q=q.squeeze(0), k=kv[0].squeeze(0), v=kv[1].squeeze(0), cu_seqlens_q=cu_seqlens_q,
        cu_seqlens_k=cu_seqlens_k, max_seqlen_q=max_seqlen_q, max_seqlen_k=max_seqlen_k,
        softmax_scale=softmax_scale, causal=causal, window_size=window_size)
    merge_attn_out(global_attn_out, global_softmax_lse, out.unsqueeze(0), lse.unsqueeze(0))


def flash_attn_varlen_bwd_func(q: torch.Tensor, kv: torch.Tensor, o: torch.Tensor, softmax_lse: torch.Tensor,
                               do: torch.Tensor, dq: torch.Tensor, dkv: torch.Tensor,
                               cu_seqlens_q: torch.Tensor, cu_seqlens_k: torch.Tensor, max_seqlen_q,
                               max_seqlen_k, softmax_scale: float, window_size: Tuple[int, int],
                               causal: bool) -> None:
    wrapped_flash_attn_bwd_varlen(
        q=q.squeeze(0), k=kv[0].squeeze(0), v=kv[1].squeeze(0), o=o.squeeze(0),
        softmax_lse=softmax_lse.squeeze(0), do=do.squeeze(0), dq=dq.squeeze(0), dk=dkv[0].squeeze(0),
        dv=dkv[1].squeeze(0), cu_seqlens_q=cu_seqlens_q, cu_seqlens_k=cu_seqlens_k, max_seqlen_q=max_seqlen_q,
        max_seqlen_k=max_seqlen_k, softmax_scale=softmax_scale, causal=causal, window_size=window_size)
