"""Host logic of ring_swa.ops.wrap_flash: the placement of queries and keys on the position axis
reproduces flash-attn's (left, right, causal) band for every shape.  No GPU needed."""
import itertools

import torch

from flash_band import band


def test_band_placement_equals_flash_definition():
    from ring_swa.ops.wrap_flash import _band
    shapes = [(1, 1), (7, 7), (5, 12), (12, 5), (16, 3), (3, 16)]
    windows = [(-1, -1), (-1, 0), (0, 0), (3, 0), (0, 4), (2, 3), (50, 50), (4, -1), (0, 16), (100, 0)]
    for (sq, sk), w, causal in itertools.product(shapes, windows, (False, True)):
        window, q0, k0 = _band(sq, sk, w, causal)
        assert window >= 0 and q0 >= 0 and k0 >= 0
        p = torch.arange(sq)[:, None] + q0
        t = torch.arange(sk)[None, :] + k0
        got = (t <= p) & (p - t <= window)
        assert torch.equal(got, band(sq, sk, w, causal)), ((sq, sk), w, causal)


def test_ops_module_exports_the_reference_names():
    import ring_swa.ops as ops
    names = ["ring_attn_p2p_communicate", "broadcast_tensor_to_group", "reduce_sum_tesnsor_to_rank",
             "exchange_and_sum_tensors", "wrapped_flash_attn_fwd", "wrapped_flash_attn_fwd_varlen",
             "wrapped_flash_attn_bwd", "wrapped_flash_attn_bwd_varlen", "flash_attn_fwd_func", "flash_attn_bwd_func",
             "flash_attn_varlen_fwd_func", "flash_attn_varlen_bwd_func", "merge_attn_out",
             "get_group_local_to_global_rank_map"]   # ring_swa/ops/__init__.py:23-38
    assert sorted(ops.__all__) == sorted(names)
    for n in names:
        assert callable(getattr(ops, n))
