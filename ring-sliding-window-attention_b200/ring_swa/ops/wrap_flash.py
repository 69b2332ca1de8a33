"""The four attention operators the reference reaches flash-attn through, on librswa.so instead.

Same names, arguments and results as ring_swa/ops/wrap_flash.py:168-429: q [B,Sq,Hq,128], k/v
[B,Sk,Hkv,128] (packed [T,H,128] for the varlen pair), `window_size=(left, right)` with -1 for
"unbounded", `causal`, flash-attn's bottom-right alignment when Sq != Sk: query i sees key j iff
    i + (Sk - Sq) - left <= j <= i + (Sk - Sq) + right          (right = 0 when causal).
The kernels know one band shape -- key position <= query position and their distance <= window -- so
the band is expressed by where queries and keys are placed on the position axis (_band below).

Differences from flash-attn: head_dim is 128 only; a query row that sees no key gets a zero output
row and lse = -inf (flash-attn 2 reports +inf there); no dropout, alibi or softcap (the reference
never passes them, ring_swa/ops/wrap_flash.py:47-69).
"""
from typing import Optional, Tuple

import torch

from .. import _kernels as K

_FAR = 1 << 29  # stands for an unbounded side of the band


def _band(sq: int, sk: int, window_size: Tuple[int, int], causal: bool) -> Tuple[int, int, int]:
    """(window, q_pos_start, k_pos_start) placing queries and keys so that the kernels' band
    `t <= p and p - t <= window` equals flash-attn's (left, right, causal) band."""
    left, right = int(window_size[0]), int(window_size[1])
    if causal:
        right = 0
    reach = sq + sk if right < 0 else min(right, sq + sk)   # past Sq + Sk positions nothing changes
    depth = _FAR if left < 0 else min(left, _FAR)
    q0 = (sk - sq) + reach                        # query i sits at i + q0, key j at j + k0
    k0 = 0
    if q0 < 0:
        k0, q0 = -q0, 0
    return min(depth + reach, _FAR), q0, k0


def wrapped_flash_attn_fwd(q, k, v, softmax_scale, window_size, causal):
    """out [B,Sq,Hq,D] (dtype of q) and softmax_lse [B,Hq,Sq] float32."""
    window, q0, k0 = _band(q.shape[1], k.shape[1], window_size, causal)
    return K.fwd(q, [K.KVSpan(k, v, k0)], window, 0, float(softmax_scale), q_pos_start=q0)


def wrapped_flash_attn_bwd(q, k, v, o, softmax_lse, do, dq, dk, dv, softmax_scale, window_size, causal):
    """Writes dq, dk, dv (overwritten, not accumulated; dk/dv may be float32 or the input dtype)."""
    window, q0, k0 = _band(q.shape[1], k.shape[1], window_size, causal)
    K.bwd(q, [K.KVSpan(k, v, k0, dk=dk, dv=dv)], o, _lse3(softmax_lse), do, dq, window, 0, float(softmax_scale),
          q_pos_start=q0)


def _lse3(lse: torch.Tensor) -> torch.Tensor:
    if lse.dtype != torch.float32 or lse.stride(-1) != 1:
        lse = lse.to(torch.float32).contiguous()
    return lse


def _same_segments(cu_q: torch.Tensor, cu_k: torch.Tensor) -> bool:
    return cu_q is cu_k or (cu_q.data_ptr() == cu_k.data_ptr() and cu_q.shape == cu_k.shape)


def _segments(cu_q: torch.Tensor, cu_k: torch.Tensor):
    a, b = cu_q.tolist(), cu_k.tolist()
    if len(a) != len(b):
        raise ValueError("cu_seqlens_q and cu_seqlens_k must describe the same number of sequences")
    return [(a[i], a[i + 1], b[i], b[i + 1]) for i in range(len(a) - 1)]


def wrapped_flash_attn_fwd_varlen(q, k, v, softmax_scale, window_size, cu_seqlens_q, cu_seqlens_k,
                                  max_seqlen_q, max_seqlen_k, causal):
    """Packed sequences: q [Tq,Hq,D], k/v [Tk,Hkv,D]; out [Tq,Hq,D], softmax_lse [Hq,Tq] float32.

    With one set of boundaries for queries and keys and nothing visible to the right (the diagonal
    call of the reference, ring_swa/sliding_window/varlen.py:120-140) this is one kernel launch over the
    packed axis.  Otherwise each sequence is its own launch with its own bottom-right alignment,
    which costs one host read of the boundaries.
    """
    Tq, Hq, D = q.shape
    out = torch.empty_like(q)
    lse = torch.empty((Hq, Tq), dtype=torch.float32, device=q.device)
    left, right = int(window_size[0]), int(window_size[1])
    if _same_segments(cu_seqlens_q, cu_seqlens_k) and (causal or right == 0):
        window = _FAR if left < 0 else left
        K.fwd(q[None], [K.KVSpan(k[None], v[None], 0)], window, 0, float(softmax_scale),
              cu_seqlens=cu_seqlens_q.to(torch.int32), out=out[None], lse=lse[None])
        return out, lse
    for q_a, q_b, k_a, k_b in _segments(cu_seqlens_q, cu_seqlens_k):
        if q_b <= q_a:
            continue
        if k_b <= k_a:
            out[q_a:q_b].zero_()
            lse[:, q_a:q_b].fill_(float("-inf"))
            continue
        window, q0, k0 = _band(q_b - q_a, k_b - k_a, window_size, causal)
        K.fwd(q[None, q_a:q_b], [K.KVSpan(k[None, k_a:k_b], v[None, k_a:k_b], k0)], window, 0, float(softmax_scale),
              q_pos_start=q0, out=out[None, q_a:q_b], lse=lse[None, :, q_a:q_b])
    return out, lse


def wrapped_flash_attn_bwd_varlen(q, k, v, o, softmax_lse, do, dq, dk, dv, softmax_scale, window_size,
                                  cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, causal):
    """Packed counterpart of wrapped_flash_attn_bwd; softmax_lse is [Hq,Tq]."""
    left, right = int(window_size[0]), int(window_size[1])
    lse = _lse3(softmax_lse)
    if _same_segments(cu_seqlens_q, cu_seqlens_k) and (causal or right == 0):
        window = _FAR if left < 0 else left
        K.bwd(q[None], [K.KVSpan(k[None], v[None], 0, dk=dk[None], dv=dv[None])], o[None], lse[None], do[None],
              dq[None], window, 0, float(softmax_scale), cu_seqlens=cu_seqlens_q.to(torch.int32))
        return
    for q_a, q_b, k_a, k_b in _segments(cu_seqlens_q, cu_seqlens_k):
        if k_b <= k_a:
            if q_b > q_a:
                dq[q_a:q_b].zero_()
            continue
        if q_b <= q_a:
            dk[k_a:k_b].zero_()
            dv[k_a:k_b].zero_()
            continue
        window, q0, k0 = _band(q_b - q_a, k_b - k_a, window_size, causal)
        span = K.KVSpan(k[None, k_a:k_b], v[None, k_a:k_b], k0, dk=dk[None, k_a:k_b], dv=dv[None, k_a:k_b])
        K.bwd(q[None, q_a:q_b], [span], o[None, q_a:q_b], lse[None, :, q_a:q_b], do[None, q_a:q_b],
              dq[None, q_a:q_b], window, 0, float(softmax_scale), q_pos_start=q0)
