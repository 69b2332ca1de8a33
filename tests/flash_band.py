"""Dense float32 restatement of the attention band flash-attn defines (test infrastructure).

Query i of Sq sees key j of Sk iff  i + (Sk - Sq) - left <= j <= i + (Sk - Sq) + right, with -1
meaning unbounded and causal forcing right = 0 -- the semantics the reference pins at its flash
boundary with test/test_local_swa.py:7-95 (window (50, 50), Sq == Sk).  Written straight from that
definition, independently of the position mapping the product uses.
"""
import torch


def band(sq, sk, window_size, causal):
    left, right = window_size
    if causal:
        right = 0
    i = torch.arange(sq)[:, None] + (sk - sq)
    j = torch.arange(sk)[None, :]
    m = torch.ones(sq, sk, dtype=torch.bool)
    if left >= 0:
        m &= j >= i - left
    if right >= 0:
        m &= j <= i + right
    return m


def attn(q, k, v, scale, window_size, causal):
    """q [B,Sq,Hq,D], k/v [B,Sk,Hkv,D] float32 (requires_grad allowed) -> out [B,Sq,Hq,D], lse [B,Hq,Sq].
    Rows that see no key give a zero output row and lse = -inf."""
    B, Sq, Hq, D = q.shape
    Sk, Hkv = k.shape[1], k.shape[2]
    g = Hq // Hkv
    kk = k.repeat_interleave(g, dim=2)
    vv = v.repeat_interleave(g, dim=2)
    s = torch.einsum("bqhd,bkhd->bhqk", q, kk) * scale
    m = band(Sq, Sk, window_size, causal)
    s = s.masked_fill(~m[None, None], float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    p = torch.exp(s - torch.where(torch.isinf(lse), torch.zeros_like(lse), lse)[..., None])
    p = torch.where(m[None, None], p, torch.zeros_like(p))
    out = torch.einsum("bhqk,bkhd->bqhd", p, vv)
    return out, lse


def attn_fwd_bwd(q, k, v, do, scale, window_size, causal):
    q, k, v = (t.detach().float().requires_grad_(True) for t in (q, k, v))
    out, lse = attn(q, k, v, scale, window_size, causal)
    out.backward(do.float())
    return out.detach(), lse.detach(), q.grad, k.grad, v.grad
