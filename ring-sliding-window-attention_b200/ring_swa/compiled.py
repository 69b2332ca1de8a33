"""Single-GPU attention registered as torch custom operators, for callers that trace their model.

The four public functions of this package run eager Python (planning, NCCL messages, ctypes calls).
For the single-GPU case (the reference's `cp_group=None` branch, ring_swa/sliding_window/nonvarlen.py:378-386,
where it calls flash-attn's registered custom ops, flash_attn_interface.py:76-133) this module offers
the same arithmetic as two registered operators, `ring_swa::swa_fwd` and `ring_swa::swa_bwd`, with
fake (shape-only) implementations and an autograd formula, so that `torch.compile` treats a call as
one opaque node instead of tracing into ctypes, and so that a call can sit inside a CUDA graph
(the kernels take fixed pointers and enqueue on the current stream; the backward's scratch is an
ordinary torch allocation made during capture).

    from ring_swa.compiled import sliding_window_attn
    out = sliding_window_attn(q, k, v, window_size=1000)                       # [B, S, H, 128]
    out = sliding_window_attn(q, k, v, 4096, cu_seqlens=cu)                    # packed [T, H, 128]
    out = sliding_window_attn(q, k, v, 8192, num_sink_tokens=1)                # StreamingLLM
"""
from typing import Optional, Tuple

import torch

from . import _kernels as K


@torch.library.custom_op("ring_swa::swa_fwd", mutates_args=(), device_types="cuda")
def swa_fwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, window: int, n_sink: int, scale: float,
            cu_seqlens: Optional[torch.Tensor]) -> Tuple[torch.Tensor, torch.Tensor]:
    out, lse = K.fwd(q, [K.KVSpan(k, v, 0)], window, n_sink, scale, cu_seqlens=cu_seqlens)
    return out, lse


@swa_fwd.register_fake
def _swa_fwd_fake(q, k, v, window, n_sink, scale, cu_seqlens):
    B, S, H, D = q.shape
    return torch.empty_like(q), q.new_empty((B, H, S), dtype=torch.float32)


@torch.library.custom_op("ring_swa::swa_bwd", mutates_args=(), device_types="cuda")
def swa_bwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, out: torch.Tensor, lse: torch.Tensor,
            dout: torch.Tensor, window: int, n_sink: int, scale: float,
            cu_seqlens: Optional[torch.Tensor]) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    K.bwd(q, [K.KVSpan(k, v, 0, dk=dk, dv=dv)], out, lse, dout.contiguous(), dq, window, n_sink, scale,
          cu_seqlens=cu_seqlens)
    return dq, dk, dv


@swa_bwd.register_fake
def _swa_bwd_fake(q, k, v, out, lse, dout, window, n_sink, scale, cu_seqlens):
    return torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)


def _setup_context(ctx, inputs, output):
    q, k, v, window, n_sink, scale, cu_seqlens = inputs
    out, lse = output
    ctx.save_for_backward(q, k, v, out, lse, *([] if cu_seqlens is None else [cu_seqlens]))
    ctx.args = (window, n_sink, scale, cu_seqlens is not None)


def _backward(ctx, dout, _dlse):
    window, n_sink, scale, has_cu = ctx.args
    q, k, v, out, lse, *rest = ctx.saved_tensors
    dq, dk, dv = swa_bwd(q, k, v, out, lse, dout, window, n_sink, scale, rest[0] if has_cu else None)
    return dq, dk, dv, None, None, None, None


swa_fwd.register_autograd(_backward, setup_context=_setup_context)


def sliding_window_attn(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, window_size: int,
                        softmax_scale: Optional[float] = None, cu_seqlens: Optional[torch.Tensor] = None,
                        num_sink_tokens: int = 0) -> torch.Tensor:
    """Sliding-window (num_sink_tokens = 0) or sink + window attention on one GPU through the
    registered operators.  q [B,S,Hq,128], k/v [B,S,Hkv,128]; with cu_seqlens (int32, device) the
    tensors are packed [T,H,128].  Differentiable w.r.t. q, k, v; returns out only, like the four
    public functions."""
    if softmax_scale is None:
        softmax_scale = q.shape[-1] ** -0.5
    packed = q.dim() == 3
    if packed != (cu_seqlens is not None):
        raise ValueError("packed [T, H, D] tensors need cu_seqlens, and only they take it")
    if packed:
        q, k, v = q[None], k[None], v[None]
    out, _lse = swa_fwd(q, k, v, int(window_size), int(num_sink_tokens), float(softmax_scale), cu_seqlens)
    return out[0] if packed else out
