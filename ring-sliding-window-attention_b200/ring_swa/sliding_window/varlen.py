"""ring_sliding_window_attn_varlen: same signature as ring_swa/sliding_window/varlen.py:362-374."""
import weakref
from typing import Optional, Sequence

import torch
from torch.distributed import ProcessGroup

from .._ring import attention, ring_ctx


# Host copies of cu_seqlens tensors already seen, by tensor object: a model hands the same tensor to
# every layer of a step, and only the first of those calls has to wait for the device.  An entry is
# valid while the very same tensor object is alive and has not been written to since.
_cu_host_cache = {}


def _cu_host(cu_seqlens: torch.Tensor):
    """(python list of the cumulative lengths, whether the call had to synchronise with the device)."""
    key = id(cu_seqlens)
    hit = _cu_host_cache.get(key)
    if hit is not None and hit[0]() is cu_seqlens and hit[1] == cu_seqlens._version:
        return hit[2], False
    host = [int(x) for x in cu_seqlens.tolist()]
    if len(_cu_host_cache) > 64:
        _cu_host_cache.clear()
    _cu_host_cache[key] = (weakref.ref(cu_seqlens), cu_seqlens._version, host)
    return host, True


def _varlen_prologue(q, k, v, cu_seqlens, cp_size, cp_chunk_lens=None):
    assert q.dim() == 3 and k.dim() == 3 and v.dim() == 3, "q, k, v must be [seq_len, heads, head_dim]"
    assert q.shape[0] == k.shape[0] == v.shape[0], "Sequence length must be the same"
    assert q.shape[1] % k.shape[1] == 0, "Number of query heads must be divisible by number of key/value heads"
    # one device-to-host copy, where the reference has its own (and several more further down):
    # the global cumulative lengths drive the halo plan on the host
    cu_host, synced = _cu_host(cu_seqlens)
    if q.is_cuda and synced:
        # the copy above has synchronised with the device anyway: a good moment to look at the status word
        from .. import _kernels
        _kernels.raise_if_reported(q.device, wait=True)
    # ring_swa/sliding_window/varlen.py:401-403; evaluated before cp_group is looked at, so a
    # missing cp_size raises TypeError there as well
    if cp_chunk_lens is None:
        assert q.shape[0] == cu_host[-1] // cp_size, "cu_seqlens does not match with sequence length per rank"
    else:
        # chunks of different lengths (not in the reference, which assumes equal ones: :56-59): the lengths
        # of all ranks' chunks must add up to the packed token axis; this rank's own is checked by the plan
        assert sum(int(x) for x in cp_chunk_lens) == cu_host[-1], "cp_chunk_lens does not add up to cu_seqlens[-1]"
    if cu_seqlens.dtype != torch.int32:
        cu_seqlens = cu_seqlens.to(torch.int32)
    return cu_seqlens.contiguous(), cu_host


def ring_sliding_window_attn_varlen(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    window_size: int,
    cu_seqlens: torch.Tensor,
    cp_group: Optional[ProcessGroup] = None,
    cp_size: Optional[int] = None,
    cp_local_rank: Optional[int] = None,
    cp_prev_global_rank: Optional[int] = None,
    cp_next_global_rank: Optional[int] = None,
    softmax_scale: Optional[float] = None,
    *,
    cp_chunk_lens: Optional[Sequence[int]] = None,
) -> torch.Tensor:
    """Ring sliding window attention over packed variable-length sequences.

    q [seq_len, num_q_heads, head_dim]; k, v [seq_len, num_kv_heads, head_dim]: this rank's equal share of
    the packed token axis.  cu_seqlens holds the cumulative lengths of ALL sequences across all ranks
    ([batch_size + 1], int32, on the device).  Other arguments as in ring_sliding_window_attn.
    Returns [seq_len, num_q_heads, head_dim].

    `cp_chunk_lens` (keyword only, not in the reference): the number of tokens on every rank of the group,
    in group-rank order (host integers, the same list on every rank), for a packed token axis that is NOT
    cut into equal shares -- e.g. cut at sequence boundaries.  Rank i then holds the tokens
    [sum(lens[:i]), sum(lens[:i+1])) and seq_len is its own entry.
    """
    cu_seqlens, cu_host = _varlen_prologue(q, k, v, cu_seqlens, cp_size, cp_chunk_lens)
    ring = ring_ctx(cp_group, cp_size, cp_local_rank, cp_prev_global_rank, cp_next_global_rank, cp_chunk_lens)
    return attention(q, k, v, window_size, 0, softmax_scale, cu_seqlens, cu_host, ring)


class RingSlidingWindowAttnVarlen:
    """The reference's autograd class by name (ring_swa/sliding_window/varlen.py:19-36): `apply` takes
    its forward's positional arguments in its order; `max_seqlen` and `cp_stream` are accepted and
    not used."""

    @staticmethod
    def apply(q, k, v, window_size, cu_seqlens, max_seqlen, cp_group, cp_size, cp_local_rank,
              cp_prev_global_rank, cp_next_global_rank, cp_stream=None, softmax_scale=None):
        return ring_sliding_window_attn_varlen(q, k, v, window_size, cu_seqlens, cp_group, cp_size, cp_local_rank,
                                               cp_prev_global_rank, cp_next_global_rank, softmax_scale)
