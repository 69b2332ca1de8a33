"""CPU stand-ins for the CUDA entry points, built on the oracle.  TEST INFRASTRUCTURE ONLY.

install() rebinds ring_swa._kernels.{fwd,bwd,merge,...} so that the ring host logic (halo plan,
exchange, phase split, gradient routing) can run on gloo CPU ranks.  The product never imports
this module.
"""
import torch

from oracle.dense_attn import dense_attn, merge_partials, band_mask

TILE = 128


def _cat(spans):
    k = torch.cat([s.k for s in spans], dim=1)
    v = torch.cat([s.v for s in spans], dim=1)
    pos = torch.cat([torch.arange(s.k.shape[1], dtype=torch.int64) + s.pos_start for s in spans])
    return k, v, pos


def _cu_list(cu):
    return None if cu is None else [int(x) for x in cu.tolist()]


def fwd(q, spans, window, n_sink, scale, q_pos_start=0, cu_seqlens=None, out=None, lse=None, q_tiles=None, carry=False):
    B, S, Hq, D = q.shape
    if out is None:
        out = torch.zeros_like(q)
    if lse is None:
        lse = torch.full((B, Hq, S), float("-inf"), dtype=torch.float32)
    a, b = (0, S) if q_tiles is None else (min(S, q_tiles[0] * TILE), min(S, q_tiles[1] * TILE))
    if b <= a:
        return out, lse
    if not spans:
        if not carry:
            out[:, a:b] = 0
            lse[:, :, a:b] = float("-inf")
        return out, lse
    k, v, pos = _cat(spans)
    o, l = dense_attn(q[:, a:b], k, v, window, scale, n_sink, _cu_list(cu_seqlens), q_pos0=q_pos_start + a,
                      k_pos=pos)
    if carry:
        o, l = merge_partials(out[:, a:b].float(), lse[:, :, a:b], o.float(), l)
    out[:, a:b] = o.to(out.dtype)
    lse[:, :, a:b] = l
    return out, lse


def bwd_workspace(q):
    return torch.zeros(1, dtype=torch.float32)


def bwd(q, spans, out, lse, dout, dq, window, n_sink, scale, q_pos_start=0, cu_seqlens=None, workspace=None,
        flags=3):
    """dk/dv of the spans that carry gradient buffers; with FINISH, dq over all the spans given."""
    if workspace is None:
        workspace = bwd_workspace(q)
    B, S, Hq, D = q.shape
    dq_sum = torch.zeros(q.shape, dtype=torch.float32)
    if spans:
        k, v, pos = _cat(spans)
        g = Hq // k.shape[2]
        kr = k.float().repeat_interleave(g, dim=2)
        vr = v.float().repeat_interleave(g, dim=2)
        q_pos = torch.arange(S, dtype=torch.int64) + q_pos_start
        mask = band_mask(q_pos, pos, window, n_sink, _cu_list(cu_seqlens))
        s = torch.einsum("bihd,bjhd->bhij", q.float(), kr) * scale
        p = torch.exp(s - lse.float()[..., None])
        p = torch.where(mask[None, None], p, torch.zeros_like(p))
        dof = dout.float()
        dp = torch.einsum("bihd,bjhd->bhij", dof, vr)
        delta = (dof * out.float()).sum(-1).permute(0, 2, 1)
        ds = p * (dp - delta[..., None])
        dq_sum = torch.einsum("bhij,bjhd->bihd", ds, kr) * scale
        dk = (torch.einsum("bhij,bihd->bjhd", ds, q.float()) * scale).reshape(B, -1, k.shape[2], g, D).sum(3)
        dv = torch.einsum("bhij,bihd->bjhd", p, dof).reshape(B, -1, k.shape[2], g, D).sum(3)
        off = 0
        for sp in spans:
            n = sp.k.shape[1]
            if sp.dk is not None:
                sp.dk.copy_(dk[:, off:off + n].to(sp.dk.dtype))
                sp.dv.copy_(dv[:, off:off + n].to(sp.dv.dtype))
            off += n
    if flags & 2:
        dq.copy_(dq_sum.to(dq.dtype))
    return workspace


def merge(o_a, lse_a, o_b, lse_b, out=None, lse_out=None):
    o, l = merge_partials(o_a.float(), lse_a, o_b.float(), lse_b)
    out = o_a if out is None else out
    lse_out = lse_a if lse_out is None else lse_out
    out.copy_(o.to(out.dtype))
    lse_out.copy_(l)
    return out, lse_out


def halo_accumulate(acc, recv):
    acc += recv.float()


def halo_accumulate_cast(dst, acc, recv):
    dst.copy_((acc + recv.float()).to(dst.dtype))


def cast_from_f32(dst, src):
    dst.copy_(src.to(dst.dtype))


def install():
    import ring_swa._kernels as K
    K.fwd, K.bwd, K.merge = fwd, bwd, merge
    K.bwd_workspace, K.halo_accumulate, K.cast_from_f32 = bwd_workspace, halo_accumulate, cast_from_f32
    K.halo_accumulate_cast = halo_accumulate_cast
