"""CPU oracle for ring sliding-window / StreamingLLM attention.  TEST INFRASTRUCTURE ONLY.

This module is the checker the CUDA path is compared against; it is never the
thing that ships or is measured as the product.  Only the test-suite, the smoke
check and the benchmark's CPU-baseline leg may import it.

It restates, in dense torch on the CPU, the reference's own dense test oracles

  * test/test_local_swa.py:7-95   torch_sliding_window_attn_nonvarlen
  * test/test_local_slm.py:7-73   torch_streaming_llm_attn_nonvarlen

generalised to what the four public ring functions compute globally (the
reference's ring schedule, ring_swa/sliding_window/nonvarlen.py:70-150 and
siblings, is a decomposition of exactly this mask):

  allowed(p, t) = same_sequence(p, t) and t <= p and
                  (p - t <= W  or  t < seq_start(p) + n_sink)

with n_sink = 0 for sliding-window attention and n_sink = 1 for StreamingLLM
(ring_swa/streaming_llm/nonvarlen.py:48-51: the sink is the first token).

Parity status: pinned.  tests/test_oracle_golden.py checks this file against
vectors produced by the reference's own code (tests/golden/make_golden.py).
"""
from __future__ import annotations

import math
from typing import Optional, Sequence, Tuple

import torch


def seq_bounds(
    positions: torch.Tensor, cu_seqlens: Optional[Sequence[int]]
) -> Tuple[torch.Tensor, torch.Tensor]:
    """Start and end (exclusive) of the sequence each global position lies in."""
    if cu_seqlens is None:
        big = torch.iinfo(torch.int64).max
        return torch.zeros_like(positions), torch.full_like(positions, big)
    cu = torch.as_tensor(list(cu_seqlens), dtype=torch.int64)
    idx = torch.searchsorted(cu, positions, right=True) - 1
    idx = idx.clamp_(0, cu.numel() - 2)
    return cu[idx], cu[idx + 1]


def band_mask(
    q_pos: torch.Tensor,
    k_pos: torch.Tensor,
    window: int,
    n_sink: int = 0,
    cu_seqlens: Optional[Sequence[int]] = None,
) -> torch.Tensor:
    """Boolean [len(q_pos), len(k_pos)] mask, True where key is visible.

    Follows test/test_local_swa.py:56-89 (lower bound ``j - i >= -W``, upper
    bound ``j <= i``) and test/test_local_slm.py:62-64 (sink column forced on),
    stated on global positions so that it also covers varlen and ring shards.
    """
    q_pos = q_pos.to(torch.int64)
    k_pos = k_pos.to(torch.int64)
    qs, _qe = seq_bounds(q_pos, cu_seqlens)
    ks, _ke = seq_bounds(k_pos, cu_seqlens)
    p = q_pos[:, None]
    t = k_pos[None, :]
    same = qs[:, None] == ks[None, :]
    causal = t <= p
    in_window = (p - t) <= window
    is_sink = t < (qs[:, None] + n_sink)
    return same & causal & (in_window | is_sink)


def dense_attn(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    window: int,
    softmax_scale: Optional[float] = None,
    n_sink: int = 0,
    cu_seqlens: Optional[Sequence[int]] = None,
    q_pos0: int = 0,
    k_pos0: int = 0,
    compute_dtype: torch.dtype = torch.float32,
    k_pos: Optional[torch.Tensor] = None,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """Dense masked softmax attention.  q [B,Sq,Hq,D], k/v [B,Sk,Hkv,D].

    Returns (out [B,Sq,Hq,D], lse [B,Hq,Sq]) in ``compute_dtype``; lse is the
    natural-log sum of exp(scale * q.k) over visible keys (-inf if none).
    Query i sits at global position q_pos0 + i; key j at k_pos0 + j, or at k_pos[j] when the
    keys are a concatenation of spans (halo, sink) that is not contiguous in position.
    Differentiable, so grads come from autograd on the same graph.
    """
    B, Sq, Hq, D = q.shape
    _, Sk, Hkv, _ = k.shape
    if softmax_scale is None:
        softmax_scale = D ** (-0.5)
    g = Hq // Hkv
    qf, kf, vf = (x.to(compute_dtype) for x in (q, k, v))
    if g != 1:  # GQA by head repetition, test/test_local_swa.py:43-49
        kf = kf.repeat_interleave(g, dim=2)
        vf = vf.repeat_interleave(g, dim=2)
    q_pos = torch.arange(Sq, dtype=torch.int64) + q_pos0
    if k_pos is None:
        k_pos = torch.arange(Sk, dtype=torch.int64) + k_pos0
    mask = band_mask(q_pos, k_pos, window, n_sink, cu_seqlens)
    s = torch.einsum("bihd,bjhd->bhij", qf, kf) * softmax_scale
    s = s.masked_fill(~mask[None, None], float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    safe = torch.where(torch.isinf(lse), torch.zeros_like(lse), lse)
    p = torch.exp(s - safe[..., None])
    p = torch.where(mask[None, None], p, torch.zeros_like(p))
    out = torch.einsum("bhij,bjhd->bihd", p, vf)
    return out, lse


def dense_attn_fwd_bwd(q, k, v, do, window, softmax_scale=None, n_sink=0,
                       cu_seqlens=None, q_pos0=0, k_pos0=0,
                       compute_dtype=torch.float32):
    """Forward + autograd backward.  Returns out, lse, dq, dk, dv (compute dtype)."""
    qf = q.detach().to(compute_dtype).requires_grad_(True)
    kf = k.detach().to(compute_dtype).requires_grad_(True)
    vf = v.detach().to(compute_dtype).requires_grad_(True)
    out, lse = dense_attn(qf, kf, vf, window, softmax_scale, n_sink, cu_seqlens,
                          q_pos0, k_pos0, compute_dtype)
    out.backward(do.to(compute_dtype))
    return out.detach(), lse.detach(), qf.grad, kf.grad, vf.grad


def merge_partials(o_a, lse_a, o_b, lse_b):
    """LSE merge of two partial attention results (ring_swa/ops/merge.py:16-50).

    o_* [B,S,H,D], lse_* [B,H,S].  (-inf, -inf) merges to (0, -inf).
    """
    lse = torch.logaddexp(lse_a, lse_b)
    wa = torch.exp(lse_a - lse)
    wb = torch.exp(lse_b - lse)
    wa = torch.where(torch.isnan(wa), torch.zeros_like(wa), wa)
    wb = torch.where(torch.isnan(wb), torch.zeros_like(wb), wb)
    o = o_a * wa.movedim(1, 2)[..., None] + o_b * wb.movedim(1, 2)[..., None]
    return o, lse


def in_window_pairs(seq_lens: Sequence[int], window: int, n_sink: int = 0) -> int:
    """Number of visible (query, key) pairs; the FLOP-count denominator."""
    def n(L, W):
        if L <= 0:
            return 0
        return L * (L + 1) // 2 if L <= W else W * (W + 1) // 2 + (L - W) * (W + 1)
    total = 0
    for L in seq_lens:
        if n_sink == 0:
            total += n(L, window)
        else:
            # exact count by position: keys visible to query i (0-based)
            # = |[max(0,i-W), i] U [0, min(n_sink, i+1))|
            ns = min(n_sink, L)
            # queries whose window still touches the sinks see i+1 keys
            cut = min(L, window + ns)  # i < cut -> window reaches into sinks
            total += cut * (cut + 1) // 2
            total += (L - cut) * (window + 1 + ns)
    return total


def attn_flops(seq_lens, window, n_q_heads, head_dim, n_sink=0, batch=1):
    """(fwd, bwd) FLOPs on visible pairs: 4*D*Hq*pairs and 10*D*Hq*pairs."""
    pairs = batch * in_window_pairs(seq_lens, window, n_sink)
    return 4 * head_dim * n_q_heads * pairs, 10 * head_dim * n_q_heads * pairs
